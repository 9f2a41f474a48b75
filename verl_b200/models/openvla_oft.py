"""OpenVLA-OFT: a vision-language-action policy (Prismatic VLM + parallel action decoding) on the native decoder.

The reference vendors the SimpleVLA-RL implementation on top of ``transformers`` + ``timm``
(verl/experimental/vla/models/openvla_oft/modeling_prismatic.py: vision backbone :83, projector :247, multimodal
forward :1091, ``OpenVLAForActionPrediction`` :1336 with ``generate_action_verl`` :1833 and the discrete log-prob path
``_verl_discrete_compute_logits`` :780). The same model here, on this package's kernels:

* vision backbone: one or two plain ViTs (DINOv2 + SigLIP in the fused variant) over ``patch_size`` patches, patch
  features taken from the second-to-last block and concatenated along the feature axis;
* projector: three linear layers (fused backbone) or two, GELU between them, into the language model's width;
* optional proprioceptive state: one more token from a two-layer MLP;
* language model: this package's :class:`CausalLM` (a Llama-2 layout for the released checkpoints, any preset for tests);
  the sequence is ``[BOS, patches..., (proprio), prompt tokens..., action placeholders..., STOP]``;
* parallel decoding (the "OFT" recipe): the ``num_actions_chunk * action_dim`` action positions enter the decoder as
  ZERO embeddings and ONE forward pass predicts all of them; the hidden state at position ``p - 1`` predicts position
  ``p``, and only the last ``n_action_bins`` entries of the vocabulary are action tokens (bin ``b`` <-> token
  ``vocab_size - 1 - b``); actions are bin centres in [-1, 1], un-normalised with the dataset's q01 / q99 statistics.

``generate_action`` samples an action chunk and returns tokens and their log-probs (what the rollout stores);
``action_log_probs`` recomputes log-probs and entropy of given action tokens with gradients (what the actor trains on).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .config import ModelConfig
from .transformer import CausalLM, PackedBatch
from .vision import _LayerNormW, _Lin


@dataclass
class ViTSpec:
    width: int = 1024
    depth: int = 24
    heads: int = 16
    mlp_ratio: float = 4.0
    layer_scale: bool = False  # DINOv2 multiplies both residual branches by a learned per-channel scale


@dataclass
class OpenVLAOFTConfig:
    llm: ModelConfig
    image_size: int = 224
    patch_size: int = 14
    backbones: tuple = (ViTSpec(1024, 24, 16, 4.0, True), ViTSpec(1152, 27, 16, 3.7362, False))  # DINOv2-L, SigLIP-so400m
    num_images_in_input: int = 1
    num_actions_chunk: int = 8
    action_dim: int = 7
    n_action_bins: int = 256
    proprio_dim: int = 0
    bos_token_id: int = 1
    stop_token_id: int = 2
    norm_stats: dict = field(default_factory=dict)  # {key: {"action": {"q01": [...], "q99": [...], "mask": [...]}}}

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch_size) ** 2 * self.num_images_in_input

    @property
    def vision_dim(self) -> int:
        return sum(b.width for b in self.backbones)

    @property
    def action_tokens(self) -> int:
        return self.num_actions_chunk * self.action_dim


class _ViTBlock(nn.Module):
    def __init__(self, s: ViTSpec, dtype, device):
        super().__init__()
        self.s = s
        self.norm1, self.norm2 = _LayerNormW(s.width, dtype, device), _LayerNormW(s.width, dtype, device)
        self.qkv = _Lin(s.width, 3 * s.width, True, dtype, device)
        self.proj = _Lin(s.width, s.width, True, dtype, device)
        hid = int(s.width * s.mlp_ratio)
        self.fc1, self.fc2 = _Lin(s.width, hid, True, dtype, device), _Lin(hid, s.width, True, dtype, device)
        if s.layer_scale:
            self.ls1 = nn.Parameter(torch.ones(s.width, dtype=dtype, device=device))
            self.ls2 = nn.Parameter(torch.ones(s.width, dtype=dtype, device=device))
        else:
            self.ls1 = self.ls2 = None

    def forward(self, x, cu, max_len):
        N, W = x.shape
        hd = W // self.s.heads
        qkv = self.qkv(self.norm1(x)).view(N, 3, self.s.heads, hd)
        a = ops.attention_varlen(qkv[:, 0].contiguous(), qkv[:, 1].contiguous(), qkv[:, 2].contiguous(), cu, max_len,
                                 causal=False)
        a = self.proj(a.reshape(N, W))
        x = x + (a * self.ls1 if self.ls1 is not None else a)
        m = self.fc2(F.gelu(self.fc1(self.norm2(x))))
        return x + (m * self.ls2 if self.ls2 is not None else m)


class PlainViT(nn.Module):
    """Patchify (a strided convolution written as unfold + GEMM), learned position embedding, pre-norm blocks. Returns
    the patch features of the second-to-last block, as the Prismatic backbones do."""

    def __init__(self, s: ViTSpec, image_size: int, patch: int, dtype, device):
        super().__init__()
        self.s, self.patch, self.grid = s, patch, image_size // patch
        self.patch_embed = _Lin(3 * patch * patch, s.width, True, dtype, device)
        self.pos_embed = nn.Parameter(torch.zeros(self.grid * self.grid, s.width, dtype=dtype, device=device))
        self.blocks = nn.ModuleList([_ViTBlock(s, dtype, device) for _ in range(s.depth)])

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        """images [B, 3, S, S] (already normalised for this backbone) -> [B, patches, width]."""
        B = images.shape[0]
        p, g = self.patch, self.grid
        x = images.reshape(B, 3, g, p, g, p).permute(0, 2, 4, 1, 3, 5).reshape(B * g * g, 3 * p * p)
        x = self.patch_embed(x.to(self.pos_embed.dtype)) + self.pos_embed.repeat(B, 1)
        n = g * g
        cu = torch.arange(0, (B + 1) * n, n, dtype=torch.int32, device=x.device)
        for blk in self.blocks[: max(len(self.blocks) - 1, 1)]:  # features of the second-to-last block
            x = blk(x, cu, n)
        return x.view(B, n, self.s.width)


class VisionBackbone(nn.Module):
    def __init__(self, c: OpenVLAOFTConfig, dtype, device):
        super().__init__()
        self.c = c
        self.towers = nn.ModuleList([PlainViT(s, c.image_size, c.patch_size, dtype, device) for s in c.backbones])

    def forward(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """pixel_values [B, num_images * 3 * num_backbones, S, S]: for every image, one normalised copy per backbone
        stacked along the channel axis. Returns [B, num_images * patches, vision_dim]."""
        nb = len(self.towers)
        per_image = pixel_values.split(3 * nb, dim=1)
        feats = []
        for img in per_image:
            feats.append(torch.cat([t(img[:, 3 * i : 3 * i + 3]) for i, t in enumerate(self.towers)], dim=-1))
        return torch.cat(feats, dim=1)


class Projector(nn.Module):
    def __init__(self, vision_dim: int, llm_dim: int, fused: bool, dtype, device):
        super().__init__()
        if fused:
            self.layers = nn.ModuleList([_Lin(vision_dim, 4 * vision_dim, True, dtype, device),
                                         _Lin(4 * vision_dim, llm_dim, True, dtype, device),
                                         _Lin(llm_dim, llm_dim, True, dtype, device)])
        else:
            self.layers = nn.ModuleList([_Lin(vision_dim, llm_dim, True, dtype, device), _Lin(llm_dim, llm_dim, True, dtype, device)])

    def forward(self, x):
        shape = x.shape
        x = x.reshape(-1, shape[-1])
        for i, l in enumerate(self.layers):
            x = l(x)
            if i + 1 < len(self.layers):
                x = F.gelu(x)
        return x.view(*shape[:-1], -1)


class OpenVLAForActionPrediction(nn.Module):
    def __init__(self, c: OpenVLAOFTConfig, dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        self.c = c
        self.vision_backbone = VisionBackbone(c, dtype, device)
        self.projector = Projector(c.vision_dim, c.llm.hidden_size, len(c.backbones) > 1, dtype, device)
        self.proprio_projector = (nn.ModuleList([_Lin(c.proprio_dim, c.llm.hidden_size, True, dtype, device),
                                                 _Lin(c.llm.hidden_size, c.llm.hidden_size, True, dtype, device)])
                                  if c.proprio_dim else None)
        self.language_model = CausalLM(c.llm, dtype=dtype, device=device)
        n = c.n_action_bins
        edges = torch.linspace(-1.0, 1.0, n)
        self.register_buffer("bin_centers", (edges[:-1] + edges[1:]) / 2.0, persistent=False)  # n - 1 centres, as OpenVLA

    def init_weights(self, seed: int = 0):
        self.language_model.init_weights(seed)
        g = torch.Generator(device=self.bin_centers.device)
        g.manual_seed(seed + 1)
        with torch.no_grad():
            for mod in (self.vision_backbone, self.projector, self.proprio_projector):
                if mod is None:
                    continue
                for name, p in mod.named_parameters():
                    if p.dim() == 2:
                        p.copy_(torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0.0, 0.02, generator=g))
        return self

    # ------------------------------------------------------------------ sequence assembly
    def _layout(self, prompt_lens: torch.Tensor):
        """Per sample: [BOS] [patches (+ proprio)] [prompt tokens without BOS] [action placeholders] [STOP]."""
        c = self.c
        n_vis = c.num_patches + (1 if c.proprio_dim else 0)
        total = prompt_lens + n_vis + c.action_tokens + 1
        return n_vis, total

    def _embed(self, input_ids, attention_mask, pixel_values, proprio):
        """Packed embeddings of the multimodal sequences. ``input_ids`` [B, L] right-padded prompts starting with BOS.
        Returns (PackedBatch, index of the first action position of every sample in the packed stream)."""
        c = self.c
        lm = self.language_model
        B = input_ids.shape[0]
        dev = input_ids.device
        lens = attention_mask.sum(-1).long()
        n_vis, total = self._layout(lens)
        vis = self.projector(self.vision_backbone(pixel_values))          # [B, patches, H]
        if self.proprio_projector is not None:
            p = self.proprio_projector[1](F.gelu(self.proprio_projector[0](proprio.to(vis.dtype))))
            vis = torch.cat([vis, p[:, None]], dim=1)
        H = vis.shape[-1]
        tok_emb = ops.embedding(input_ids.reshape(-1), lm.embed_tokens.weight).view(B, -1, H)
        stop = ops.embedding(torch.full((1,), c.stop_token_id, device=dev, dtype=torch.long), lm.embed_tokens.weight)[0]
        pieces, ids, first_action = [], [], []
        off = 0
        for b in range(B):
            L = int(lens[b])
            zeros = torch.zeros(c.action_tokens, H, dtype=vis.dtype, device=dev)  # parallel decoding: empty action slots
            pieces += [tok_emb[b, :1], vis[b].to(tok_emb.dtype), tok_emb[b, 1:L], zeros.to(tok_emb.dtype), stop[None]]
            ids.append(torch.cat([input_ids[b, :1], torch.zeros(n_vis, dtype=torch.long, device=dev), input_ids[b, 1:L],
                                  torch.zeros(c.action_tokens, dtype=torch.long, device=dev),
                                  torch.full((1,), c.stop_token_id, dtype=torch.long, device=dev)]))
            first_action.append(off + 1 + n_vis + (L - 1))
            off += int(total[b])
        emb = torch.cat(pieces, dim=0)
        cu = F.pad(total.cumsum(0), (1, 0)).to(torch.int32)
        pos = torch.cat([torch.arange(int(t), device=dev) for t in total])
        batch = PackedBatch(torch.cat(ids), pos, cu, int(total.max()), inputs_embeds=emb)
        return batch, torch.tensor(first_action, device=dev)

    def _action_logits(self, input_ids, attention_mask, pixel_values, proprio=None, temperature: float = 1.0):
        """fp32 logits over the action bins for every action position: [B, action_tokens, n_action_bins]. Column j is
        bin j (token ``vocab_size - 1 - j``)."""
        c = self.c
        batch, first = self._embed(input_ids, attention_mask, pixel_values, proprio)
        hidden = self.language_model.forward_hidden(batch)
        # the hidden state one position earlier predicts each action token
        idx = (first[:, None] - 1 + torch.arange(c.action_tokens, device=first.device)[None]).reshape(-1)
        h = hidden[idx]
        V = c.llm.vocab_size
        w = self.language_model.lm_head_weight[V - c.n_action_bins :]       # the action tokens are the last rows
        logits = (h.float() @ w.float().t()) if not h.is_cuda else ops.gemm(h.contiguous(), w.contiguous(), out_dtype=torch.float32)
        logits = logits.flip(-1)                                            # row V - 1 - j -> column j
        return logits.view(input_ids.shape[0], c.action_tokens, c.n_action_bins) / max(float(temperature), 1e-6)

    # ------------------------------------------------------------------ rollout and training interfaces
    def bins_to_actions(self, bins: torch.Tensor) -> torch.Tensor:
        """Bin indices [B, action_tokens] -> normalised actions [B, chunk, action_dim] in [-1, 1]."""
        centers = self.bin_centers.to(bins.device)
        a = centers[bins.clamp(max=centers.numel() - 1)]
        return a.view(bins.shape[0], self.c.num_actions_chunk, self.c.action_dim)

    def unnormalize(self, actions: torch.Tensor, unnorm_key: Optional[str] = None) -> torch.Tensor:
        """[-1, 1] -> the robot's units with the dataset's 1st / 99th percentiles (dimensions with mask = False, e.g. the
        gripper, pass through)."""
        if not self.c.norm_stats:
            return actions
        key = unnorm_key or next(iter(self.c.norm_stats))
        st = self.c.norm_stats[key]["action"]
        lo = torch.tensor(st["q01"], dtype=actions.dtype, device=actions.device)
        hi = torch.tensor(st["q99"], dtype=actions.dtype, device=actions.device)
        mask = torch.tensor(st.get("mask", [True] * lo.numel()), device=actions.device)
        return torch.where(mask, 0.5 * (actions + 1.0) * (hi - lo) + lo, actions)

    @torch.no_grad()
    def generate_action(self, input_ids, attention_mask, pixel_values, proprio=None, temperature: float = 1.0,
                        do_sample: bool = True, generator: Optional[torch.Generator] = None, unnorm_key: Optional[str] = None):
        """One forward pass for a whole action chunk. Returns dict(actions [B, chunk, dim] un-normalised,
        normalized_actions, responses = action token ids [B, action_tokens], log_probs [B, action_tokens])."""
        logits = self._action_logits(input_ids, attention_mask, pixel_values, proprio, temperature if do_sample else 1.0)
        logp = torch.log_softmax(logits, -1)
        if do_sample:
            flat = logp.exp().reshape(-1, logp.shape[-1])
            bins = torch.multinomial(flat.cpu() if generator is not None and generator.device.type == "cpu" else flat, 1,
                                     generator=generator).to(logp.device).view(logp.shape[:2])
        else:
            bins = logp.argmax(-1)
        lp = logp.gather(-1, bins[..., None])[..., 0]
        norm = self.bins_to_actions(bins)
        return {"actions": self.unnormalize(norm, unnorm_key), "normalized_actions": norm,
                "responses": self.c.llm.vocab_size - 1 - bins, "log_probs": lp}

    def action_log_probs(self, input_ids, attention_mask, pixel_values, responses, proprio=None, temperature: float = 1.0):
        """Log-probs [B, action_tokens] and entropies of the action tokens ``responses`` (with gradients)."""
        logits = self._action_logits(input_ids, attention_mask, pixel_values, proprio, temperature)
        logp = torch.log_softmax(logits, -1)
        bins = (self.c.llm.vocab_size - 1 - responses).clamp(0, self.c.n_action_bins - 1)
        ent = -(logp.exp() * logp).sum(-1)
        return logp.gather(-1, bins[..., None])[..., 0], ent


class OpenVLAPolicy:
    """Adapter for :class:`verl_b200.experimental.vla.env_loop.EnvLoop`: observations (images uint8 [E, S, S, 3], task
    strings) -> (action tokens as bin indices [E, action_tokens], log-probs). ``tokenize(task) -> list[int]`` turns the
    instruction into prompt ids (BOS first); images are resized to the model's input size and normalised per backbone."""

    def __init__(self, model: OpenVLAForActionPrediction, tokenize, temperature: float = 1.0, seed: int = 0,
                 means=((0.485, 0.456, 0.406), (0.5, 0.5, 0.5)), stds=((0.229, 0.224, 0.225), (0.5, 0.5, 0.5))):
        self.model, self.tokenize, self.temperature = model, tokenize, temperature
        self.gen = torch.Generator().manual_seed(seed)
        self.means, self.stds = means, stds
        self.last_inputs = None

    def preprocess(self, images) -> torch.Tensor:
        c = self.model.c
        x = torch.as_tensor(images).permute(0, 3, 1, 2).float() / 255.0
        if x.shape[-1] != c.image_size:
            x = F.interpolate(x, size=(c.image_size, c.image_size), mode="bilinear", align_corners=False)
        outs = []
        for i in range(len(c.backbones)):
            m = torch.tensor(self.means[i % len(self.means)]).view(1, 3, 1, 1)
            s = torch.tensor(self.stds[i % len(self.stds)]).view(1, 3, 1, 1)
            outs.append((x - m) / s)
        return torch.cat(outs, dim=1)

    def inputs(self, obs: dict):
        prompts = [self.tokenize(f"In: What action should the robot take to {t.lower()}?\nOut:") for t in obs["task"]]
        L = max(len(p) for p in prompts)
        ids = torch.zeros(len(prompts), L, dtype=torch.long)
        mask = torch.zeros(len(prompts), L, dtype=torch.long)
        for i, p in enumerate(prompts):
            ids[i, : len(p)] = torch.tensor(p)
            mask[i, : len(p)] = 1
        dev = next(self.model.parameters()).device
        return ids.to(dev), mask.to(dev), self.preprocess(obs["images"]).to(dev)

    @torch.no_grad()
    def __call__(self, obs: dict):
        ids, mask, pix = self.inputs(obs)
        out = self.model.generate_action(ids, mask, pix, temperature=self.temperature, generator=self.gen)
        self.last_inputs = (ids, mask, pix)
        bins = self.model.c.llm.vocab_size - 1 - out["responses"]
        return bins.cpu().numpy(), out["log_probs"].float().cpu().numpy()
