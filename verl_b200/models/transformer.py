"""Decoder-only transformer (Llama / Qwen2 / Qwen3 / Qwen3-MoE families) written against
:mod:`verl_b200.ops`, operating on packed (remove-padding) token streams.

The reference takes these models from HF ``transformers`` and monkey-patches attention and the
lm_head (verl/models/transformers/monkey_patch.py:286-493, dense_common.py:72-193). Here the
layer is a short sequence of native ops:

    rmsnorm(+residual) -> qkv GEMM(+bias) -> [q/k norm] -> RoPE -> varlen causal GQA attention
    -> o GEMM -> rmsnorm(+residual) -> gate|up GEMM -> SwiGLU -> down GEMM

q/k/v and gate/up weights are stored fused ([q;k;v] rows, [gate;up] rows); HF checkpoints are
split/merged by :mod:`verl_b200.models.hf_io`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .config import ModelConfig


@dataclass
class PackedBatch:
    """Inputs of one packed forward: T tokens from B sequences."""

    input_ids: torch.Tensor  # [T] int64
    position_ids: torch.Tensor  # [T] int64
    cu_seqlens: torch.Tensor  # [B+1] int32
    max_seqlen: int
    total_tokens: int = -1  # Ulysses: tokens of the whole packed stream when input_ids holds only this rank's slice
    # vision-language models: patches of all images of the batch (in order) and their (t, h, w) grids; position_ids is
    # then [3, T] (multimodal RoPE)
    pixel_values: Optional[torch.Tensor] = None
    image_grid_thw: Optional[torch.Tensor] = None
    # the same for videos (grids with t > 1: one attention segment per frame group); their outputs fill the video
    # placeholder tokens
    pixel_values_videos: Optional[torch.Tensor] = None
    video_grid_thw: Optional[torch.Tensor] = None
    # embeddings computed by the caller ([T, H]; vision-language-action models splice projected image patches and
    # action placeholders into the token stream themselves): used instead of the embedding lookup
    inputs_embeds: Optional[torch.Tensor] = None
    # shared-prefix evaluation (forward only): the stream holds every distinct prompt ONCE, then all responses; a
    # response attends to its prompt's keys and to itself. dict(n_prompt_tokens, cu_prompt, max_prompt, cu_resp,
    # max_resp, k_gather [sum(prompt + response lengths)], cu_k, max_k): see trainer/ppo/prefix_grouper_utils.py
    prefix_share: Optional[dict] = None

    @classmethod
    def from_padded(cls, input_ids: torch.Tensor, attention_mask: torch.Tensor, position_ids: torch.Tensor | None = None):
        """Remove padding from [B,S] inputs. Returns (batch, flat_indices) where flat_indices are the
        positions of the kept tokens in the flattened [B*S] layout (for scattering outputs back)."""
        mask = attention_mask.bool()
        seqlens = mask.sum(-1).int()
        idx = torch.nonzero(mask.flatten(), as_tuple=False).flatten()
        ids = input_ids.flatten()[idx]
        if position_ids is None:
            position_ids = (torch.cumsum(mask.long(), -1) - 1).clamp(min=0)
        if position_ids.dim() == 3:  # [B, 3, S] multimodal RoPE positions -> [3, T]
            pos = torch.stack([position_ids[:, a].flatten()[idx] for a in range(position_ids.shape[1])])
        else:
            pos = position_ids.flatten()[idx]
        cu = torch.zeros(seqlens.numel() + 1, dtype=torch.int32, device=input_ids.device)
        cu[1:] = torch.cumsum(seqlens, 0)
        return cls(ids, pos, cu, int(seqlens.max().item()) if seqlens.numel() else 0), idx


class Linear(nn.Module):
    def __init__(self, in_f: int, out_f: int, bias: bool, dtype, device, std: float = 0.02):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_f, in_f, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_f, dtype=dtype, device=device)) if bias else None
        self._std = std

    def reset_parameters(self, generator=None):
        with torch.no_grad():
            self.weight.copy_(
                torch.empty(self.weight.shape, dtype=torch.float32, device=self.weight.device).normal_(
                    0.0, self._std, generator=generator))
            if self.bias is not None:
                self.bias.zero_()

    def forward(self, x):
        y = ops.linear(x, self.weight, self.bias)
        a = self.__dict__.get("lora_A")
        if a is not None and not self.__dict__.get("lora_off", False):  # LoRA branch (models/lora.py): fp32 adapters, cast at use
            y = y + self.lora_scale * ops.linear(ops.linear(x, a.to(x.dtype)), self.lora_B.to(x.dtype))
        return y


class RMSNormWeight(nn.Module):
    def __init__(self, dim: int, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))


class DenseMLP(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.gate_up_proj = Linear(cfg.hidden_size, 2 * cfg.intermediate_size, False, dtype, device)
        self.down_proj = Linear(cfg.intermediate_size, cfg.hidden_size, False, dtype, device)
        self.tile_shards = 1  # >1: run over row shards with per-shard recomputation (models/tiled_mlp.py)
        self.tp_group = None  # training-side tensor parallelism: this module holds a column / row slice of the MLP

    def _plain(self, x):
        if self.tp_group is not None:
            from ..parallel.tensor_parallel import copy_to_tp_region, reduce_from_tp_region

            x = copy_to_tp_region(x, self.tp_group)
            return reduce_from_tp_region(self.down_proj(ops.swiglu(self.gate_up_proj(x))), self.tp_group)
        return self.down_proj(ops.swiglu(self.gate_up_proj(x)))

    def forward(self, x):
        if self.tile_shards > 1:
            from .tiled_mlp import tiled_call

            return tiled_call(self._plain, [self.gate_up_proj.weight, self.down_proj.weight], self.tile_shards, x)
        return self._plain(x)


class XieluMLP(nn.Module):
    """Apertus: ``down(xielu(up(x)))`` with xielu(v) = alpha_p v^2 + beta v for v > 0 and
    alpha_n (expm1(min(v, eps)) - v) + beta v otherwise; alpha_p = softplus(a_p), alpha_n = beta + softplus(a_n) with one
    learnable (a_p, a_n) pair per layer (transformers' ``ApertusMLP`` / ``XIELUActivation``; the reference serves the
    family through verl/models/transformers/apertus.py)."""

    BETA, EPS = 0.5, -1e-6

    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.up_proj = Linear(cfg.hidden_size, cfg.intermediate_size, False, dtype, device)
        self.down_proj = Linear(cfg.intermediate_size, cfg.hidden_size, False, dtype, device)
        init = math.log(math.expm1(0.8))
        self.act_alpha_p = nn.Parameter(torch.full((1,), init, dtype=dtype, device=device))
        self.act_alpha_n = nn.Parameter(torch.full((1,), math.log(math.expm1(0.8 - self.BETA)), dtype=dtype, device=device))
        self.tp_group = None

    def forward(self, x):
        v = self.up_proj(x).float()
        ap = F.softplus(self.act_alpha_p.float())
        an = self.BETA + F.softplus(self.act_alpha_n.float())
        neg = (torch.expm1(torch.clamp(v, max=self.EPS)) - v) * an + self.BETA * v
        h = torch.where(v > 0, ap * v * v + self.BETA * v, neg)
        return self.down_proj(h.to(x.dtype))


class MoEMLP(nn.Module):
    """Top-k routed experts (Qwen3-MoE): softmax router, top-k, optional renormalisation.

    Tokens are sorted by expert and each expert's slice goes through the GEMM kernels;
    ``last_routing`` keeps (top-k ids, weights) of the latest forward for router replay
    (verl/utils/megatron/router_replay_utils.py)."""

    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.E, self.k = cfg.num_experts, cfg.num_experts_per_tok
        self.norm_topk = cfg.norm_topk_prob
        I, H = cfg.moe_intermediate_size, cfg.hidden_size
        # expert parallelism over replicated tokens (a tensor-parallel rollout replica): this module holds the experts
        # [e_off, e_off + E_local) and returns its partial sum; the caller adds the ranks' results up
        ep, ep_rank = int(cfg.extra.get("ep_size", 1) or 1), int(cfg.extra.get("ep_rank", 0) or 0)
        assert self.E % ep == 0, f"{self.E} experts are not divisible by expert-parallel size {ep}"
        self.E_local, self.e_off = self.E // ep, ep_rank * (self.E // ep)
        self.gate = Linear(H, self.E, False, dtype, device)
        self.gate_up_proj = nn.Parameter(torch.empty(self.E_local, 2 * I, H, dtype=dtype, device=device))
        self.down_proj = nn.Parameter(torch.empty(self.E_local, H, I, dtype=dtype, device=device))
        self.last_routing = None
        self.replay_routing = None
        self.tp_group = None  # training with the experts sharded over a tensor-parallel group (tokens replicated)
        self.ep_group = None  # training with expert parallelism: tokens travel to the rank that owns the expert

    def reset_parameters(self, generator=None):
        self.gate.reset_parameters(generator)
        with torch.no_grad():
            for p in (self.gate_up_proj, self.down_proj):
                p.copy_(torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0.0, 0.02, generator=generator))

    def forward(self, x):
        if self.tp_group is not None:
            from ..parallel.tensor_parallel import copy_to_tp_region, reduce_from_tp_region

            # every rank routes the same tokens and runs its own experts; the partial sums add up to the layer's
            # output. Through the experts every rank sees only its share of d x and of d (routing weights): those are
            # summed over the group; the router itself runs replicated on x, so its own d x is already complete.
            return reduce_from_tp_region(self._forward(copy_to_tp_region(x, self.tp_group), x), self.tp_group)
        return self._forward(x, x)

    def _forward(self, x, x_router):
        T, H = x.shape
        logits = self.gate(x_router).float()
        probs = torch.softmax(logits, dim=-1)
        if self.replay_routing is not None:
            top_i = self.replay_routing
            top_w = probs.gather(-1, top_i)
        else:
            top_w, top_i = torch.topk(probs, self.k, dim=-1)
        if self.norm_topk:
            top_w = top_w / top_w.sum(-1, keepdim=True)
        if self.tp_group is not None:
            from ..parallel.tensor_parallel import copy_to_tp_region

            top_w = copy_to_tp_region(top_w, self.tp_group)  # each rank sees only its experts' share of d top_w
        self.last_routing = top_i.detach()
        if self.ep_group is not None:
            from ..parallel.expert_parallel import ep_moe_mlp

            return ep_moe_mlp(x, top_i, top_w, self.gate_up_proj, self.down_proj, ops.swiglu, self.ep_group, self.E)
        if x.is_cuda and _grouped_gemm_ok(self.gate_up_proj, self.down_proj):
            # one grouped GEMM per projection for all experts, routing layout computed on the device
            from ..ops.moe import moe_mlp

            return moe_mlp(x, top_i, top_w, self.gate_up_proj, self.down_proj, ops.swiglu, expert_offset=self.e_off,
                           num_experts=self.E)
        flat_e = top_i.flatten()
        order = torch.argsort(flat_e, stable=True)
        tok = order // self.k
        counts = torch.bincount(flat_e, minlength=self.E).tolist()
        xs = x[tok]
        pieces = []
        start = 0
        for e, n in enumerate(counts):
            if n == 0:
                continue
            seg = xs[start : start + n]
            if self.e_off <= e < self.e_off + self.E_local:
                h = ops.swiglu(ops.linear(seg, self.gate_up_proj[e - self.e_off]))
                pieces.append(ops.linear(h, self.down_proj[e - self.e_off]))
            else:  # another rank's expert: no contribution to this rank's partial sum
                pieces.append(torch.zeros(n, H, dtype=x.dtype, device=x.device))
            start += n
        outs = torch.cat(pieces, dim=0) if pieces else torch.empty(0, H, dtype=x.dtype, device=x.device)
        w = top_w.flatten()[order].to(x.dtype).unsqueeze(-1)
        y = torch.zeros(T, H, dtype=x.dtype, device=x.device)
        y.index_add_(0, tok, outs * w)
        return y


def _grouped_gemm_ok(gate_up: torch.Tensor, down: torch.Tensor) -> bool:
    """Grouped-GEMM constraints: bf16, contraction lengths multiples of 64."""
    return (gate_up.dtype == torch.bfloat16 and gate_up.shape[1] % 64 == 0 and gate_up.shape[2] % 64 == 0
            and down.shape[1] % 64 == 0 and down.shape[2] % 64 == 0)


class Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.qkv_proj = Linear(cfg.hidden_size, cfg.q_size + 2 * cfg.kv_size, cfg.attention_bias, dtype, device)
        self.o_proj = Linear(cfg.q_size, cfg.hidden_size, False, dtype, device)
        if cfg.qk_norm:
            self.q_norm = RMSNormWeight(cfg.head_dim, dtype, device)
            self.k_norm = RMSNormWeight(cfg.head_dim, dtype, device)
        self.sp_group = None  # Ulysses sequence-parallel group (set by the engine)
        self.cp_group = None  # context-parallel group: the batch then holds this rank's two zig-zag chunks
        self.tp_group = None  # training-side tensor parallelism: this module holds 1 / tp of the heads

    def _attend(self, q, k, v, batch: PackedBatch):
        """Attention proper. Under Ulysses the inputs are this rank's sequence slice with all heads; an all-to-all
        makes them the whole sequence with a slice of the heads and another one brings the output back
        (verl/models/transformers/monkey_patch.py:87-155)."""
        if batch.prefix_share is not None:
            return self._attend_shared_prefix(q, k, v, batch.prefix_share)
        if self.cp_group is not None:
            from ..parallel.context_parallel import cp_attention

            # batch.cu_seqlens / max_seqlen describe ONE chunk of every sequence; q, k, v hold two of them
            return cp_attention(q.contiguous(), k.contiguous(), v.contiguous(), batch.cu_seqlens, batch.max_seqlen,
                                self.cp_group)
        if self.sp_group is None:
            return ops.attention_varlen(q, k, v, batch.cu_seqlens, batch.max_seqlen, causal=True)
        import torch.distributed as dist

        from ..utils.ulysses import gather_heads_scatter_seq, gather_seq_scatter_heads

        sp = dist.get_world_size(self.sp_group)
        Hk = k.shape[1]
        if Hk % sp != 0:  # fewer KV heads than ranks: replicate them so that every rank owns whole heads
            assert sp % Hk == 0, f"ulysses size {sp} and {Hk} KV heads are incompatible"
            k = k.repeat_interleave(sp // Hk, dim=1)
            v = v.repeat_interleave(sp // Hk, dim=1)
        total = batch.total_tokens if batch.total_tokens > 0 else q.shape[0] * sp
        q = gather_seq_scatter_heads(q, 0, 1, total, self.sp_group)
        k = gather_seq_scatter_heads(k, 0, 1, total, self.sp_group)
        v = gather_seq_scatter_heads(v, 0, 1, total, self.sp_group)
        o = ops.attention_varlen(q.contiguous(), k.contiguous(), v.contiguous(), batch.cu_seqlens, batch.max_seqlen, causal=True)
        return gather_heads_scatter_seq(o, 1, 0, self.sp_group)

    def _attend_shared_prefix(self, q, k, v, ps: dict):
        """Prompts (each stored once) attend to themselves causally; every response attends to the keys of ITS prompt
        followed by its own keys, causally aligned at the end (the prefix-sharing attention of the reference's
        ``use_prefix_grouper`` path, verl/trainer/ppo/prefix_grouper_utils.py). Forward only."""
        assert not (torch.is_grad_enabled() and q.requires_grad), "shared-prefix attention is a forward-only path"
        assert self.sp_group is None and self.cp_group is None, "shared-prefix attention does not combine with SP / CP"
        from ..rollout.engine import _varlen_attention_kv

        Tp = ps["n_prompt_tokens"]
        out_p = ops.attention_varlen(q[:Tp], k[:Tp], v[:Tp], ps["cu_prompt"], ps["max_prompt"], causal=True)
        k_cat, v_cat = k.index_select(0, ps["k_gather"]), v.index_select(0, ps["k_gather"])
        out_r = _varlen_attention_kv(q[Tp:], k_cat, v_cat, ps["cu_resp"], ps["cu_k"], ps["max_resp"], ps["max_k"])
        return torch.cat([out_p, out_r.to(out_p.dtype)], dim=0)

    def forward(self, x, batch: PackedBatch, rope):
        cfg = self.cfg
        Hq, Hk, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        T = x.shape[0]
        if self.tp_group is not None:
            from ..parallel.tensor_parallel import copy_to_tp_region

            x = copy_to_tp_region(x, self.tp_group)
        qkv = self.qkv_proj(x)
        if cfg.qk_norm:
            q, k, v = qkv.split([cfg.q_size, cfg.kv_size, cfg.kv_size], dim=-1)
            qw, kw = self.q_norm.weight, self.k_norm.weight
            if self.tp_group is not None:  # shared by all heads: every rank sees its own heads' share of the gradient
                qw, kw = copy_to_tp_region(qw, self.tp_group), copy_to_tp_region(kw, self.tp_group)
            q, _ = ops.rmsnorm(q.reshape(T * Hq, D), qw, cfg.rms_norm_eps)
            k, _ = ops.rmsnorm(k.reshape(T * Hk, D), kw, cfg.rms_norm_eps)
            qkv = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v], dim=-1)
        qkv = ops.rope_qkv(qkv, batch.position_ids, rope[0], rope[1], Hq, Hk, D, mrope_section=cfg.mrope_section,
                           mrope_interleaved=cfg.mrope_interleaved)
        q = qkv[:, : cfg.q_size].view(T, Hq, D)
        k = qkv[:, cfg.q_size : cfg.q_size + cfg.kv_size].view(T, Hk, D)
        v = qkv[:, cfg.q_size + cfg.kv_size :].view(T, Hk, D)
        o = self._attend(q, k, v, batch)
        out = self.o_proj(o.reshape(T, cfg.q_size))
        if self.tp_group is not None:
            from ..parallel.tensor_parallel import reduce_from_tp_region

            out = reduce_from_tp_region(out, self.tp_group)
        return out


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.input_layernorm = RMSNormWeight(cfg.hidden_size, dtype, device)
        self.self_attn = Attention(cfg, dtype, device)
        self.post_attention_layernorm = RMSNormWeight(cfg.hidden_size, dtype, device)
        self.mlp = (MoEMLP(cfg, dtype, device) if cfg.is_moe else
                    DenseMLP(cfg, dtype, device) if cfg.mlp_gated else XieluMLP(cfg, dtype, device))

    def forward(self, hidden, residual, batch: PackedBatch, rope):
        """(hidden, residual) -> (hidden, residual); the residual add is fused into the next norm."""
        eps = self.cfg.rms_norm_eps
        normed, residual = ops.rmsnorm(hidden, self.input_layernorm.weight, eps, residual)
        attn = self.self_attn(normed, batch, rope)
        normed, residual = ops.rmsnorm(attn, self.post_attention_layernorm.weight, eps, residual)
        return self.mlp(normed), residual


class CausalLM(nn.Module):
    """Packed-sequence causal LM with an lm_head (policy / reference) or a value head (critic)."""

    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", value_head: bool = False,
                 layer_range: Optional[tuple] = None, has_embed: bool = True, has_head: bool = True):
        """``layer_range = (lo, hi)``, ``has_embed``, ``has_head``: one pipeline stage of the model (decoder layers
        ``lo .. hi - 1``; the embedding lives on the first stage, final norm and head on the last). ``layers[i]`` is then
        decoder layer ``lo + i`` (``layer_offset``)."""
        super().__init__()
        self.cfg = cfg
        self.value_head = value_head or cfg.num_labels == 1
        lo, hi = layer_range if layer_range is not None else (0, cfg.num_hidden_layers)
        self.layer_offset = lo
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device) if has_embed else None
        self.layers = nn.ModuleList([DecoderLayer(cfg, dtype, device) for _ in range(lo, hi)])
        self.norm = RMSNormWeight(cfg.hidden_size, dtype, device) if has_head else None
        if not has_head:
            self.lm_head = None
        elif self.value_head:
            self.score = Linear(cfg.hidden_size, 1, False, dtype, device)
            self.lm_head = None
        elif cfg.tie_word_embeddings:
            assert has_embed, "tied embeddings need the embedding and the head on the same pipeline stage"
            self.lm_head = None
        else:
            # training-side tensor parallelism may give this rank a slice of the vocabulary rows
            self.lm_head = Linear(cfg.hidden_size, int(cfg.extra.get("lm_head_rows", cfg.vocab_size)), False, dtype, device)
        self.visual = None
        if cfg.is_vl and has_embed:
            from .vision import VisionConfig, VisionTower

            self.visual = VisionTower(VisionConfig.from_dict(cfg.extra["vision_config"]), dtype=dtype, device=device)
        self.gradient_checkpointing = False
        # training-side tensor parallelism: an untied lm_head holds a slice of the vocabulary rows
        self.tp_group = None
        self.vocab_offset = 0

    # ------------------------------------------------------------------ init
    def init_weights(self, seed: int = 0):
        dev = next(self.parameters()).device
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed)
        if self.embed_tokens is not None:
            with torch.no_grad():
                w = self.embed_tokens.weight
                w.copy_(torch.empty(w.shape, dtype=torch.float32, device=w.device).normal_(0.0, 0.02, generator=gen))
        for m in self.modules():
            if isinstance(m, (Linear, MoEMLP)):
                m.reset_parameters(gen)
        if self.visual is not None:
            self.visual.init_weights(seed + 1)
        return self

    @property
    def lm_head_weight(self) -> torch.Tensor:
        return self.embed_tokens.weight if self.lm_head is None else self.lm_head.weight

    def rope(self, device) -> tuple[torch.Tensor, torch.Tensor]:
        c = self.cfg
        return ops.rope_tables(c.head_dim, c.max_position_embeddings, c.rope_theta, device, c.extra.get("rope_scaling"))

    # --------------------------------------------------------------- forward
    @property
    def num_deepstack(self) -> int:
        """Qwen3-VL: how many of the first decoder layers get a deepstack feature of the vision tower added to the hidden
        states of the image tokens after them."""
        return self.visual.num_deepstack if self.visual is not None else 0

    def embed(self, batch: PackedBatch, with_deepstack: bool = False):
        """Token embeddings ``[T, H]`` with the vision tower's outputs at the image placeholder tokens.
        ``with_deepstack``: a tuple ``(embeddings, feature_0, ..., feature_{n-1})`` with ``n = num_deepstack``; feature i
        (``[number of image tokens, H]``, zero rows when the batch has no image) is for :meth:`add_deepstack` after
        decoder layer i."""
        n_ds = self.num_deepstack if with_deepstack else 0
        if batch.inputs_embeds is not None:
            h = batch.inputs_embeds.to(self.embed_tokens.weight.dtype)
            return (h,) + tuple(h.new_zeros(0, h.shape[1]) for _ in range(n_ds)) if with_deepstack else h
        h = ops.embedding(batch.input_ids, self.embed_tokens.weight)
        taps = [h.new_zeros(0, h.shape[1]) for _ in range(n_ds)]
        has_img = batch.pixel_values is not None and batch.pixel_values.numel() > 0
        has_vid = batch.pixel_values_videos is not None and batch.pixel_values_videos.numel() > 0
        if self.visual is not None and (has_img or has_vid):
            # the vision tower's outputs replace the embeddings of the placeholder tokens, in order: one call over the
            # images' patches followed by the videos' (every image / frame group is its own attention segment)
            pixels = [p for p, on in ((batch.pixel_values, has_img), (batch.pixel_values_videos, has_vid)) if on]
            grids = [g for g, on in ((batch.image_grid_thw, has_img), (batch.video_grid_thw, has_vid)) if on]
            pixels, grids = torch.cat(pixels, 0), torch.cat(grids, 0)
            if self.visual.num_deepstack:
                vis, feats = self.visual(pixels, grids, return_deepstack=True)
                if with_deepstack:
                    taps = [f.to(h.dtype) for f in feats]
            else:
                vis = self.visual(pixels, grids)
            where = self._vision_rows(batch)
            assert where.numel() == vis.shape[0], f"{where.numel()} placeholder tokens but {vis.shape[0]} vision embeddings"
            h = h.index_put((where,), vis.to(h.dtype))
        return (h, *taps) if with_deepstack else h

    def _vision_rows(self, batch: PackedBatch) -> torch.Tensor:
        """Rows of the image placeholder tokens followed by the rows of the video placeholder tokens: the order of the
        vision tower's outputs."""
        where = torch.nonzero(batch.input_ids == self.cfg.image_token_id, as_tuple=True)[0]
        vid = self.cfg.extra.get("video_token_id")
        if vid is not None and batch.pixel_values_videos is not None and batch.pixel_values_videos.numel():
            where = torch.cat([where, torch.nonzero(batch.input_ids == int(vid), as_tuple=True)[0]])
        return where

    def add_deepstack(self, hidden: torch.Tensor, batch: PackedBatch, feature: torch.Tensor) -> torch.Tensor:
        """``hidden`` with ``feature`` added at the rows of the vision placeholder tokens (the residual stream of a layer
        is ``hidden + residual``, so adding to ``hidden`` adds to the stream)."""
        if feature.shape[0] == 0:
            return hidden
        return hidden.index_add(0, self._vision_rows(batch), feature.to(hidden.dtype))

    def final_norm(self, hidden, residual) -> torch.Tensor:
        out, _ = ops.rmsnorm(hidden, self.norm.weight, self.cfg.rms_norm_eps, residual)
        return out

    def forward_hidden(self, batch: PackedBatch) -> torch.Tensor:
        """Final-norm hidden states [T,H] of a packed batch."""
        hidden, *taps = self.embed(batch, with_deepstack=True)
        residual = None
        rope = self.rope(hidden.device)
        for i, layer in enumerate(self.layers):
            if self.gradient_checkpointing and torch.is_grad_enabled():
                hidden, residual = torch.utils.checkpoint.checkpoint(layer, hidden, residual, batch, rope,
                                                                     use_reentrant=False)
            else:
                hidden, residual = layer(hidden, residual, batch, rope)
            if i < len(taps):
                hidden = self.add_deepstack(hidden, batch, taps[i])
        return self.final_norm(hidden, residual)

    def logprob_entropy(self, hidden: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0):
        """Per-token log-prob of ``labels`` and entropy from final hidden states (fused, no logits)."""
        if self.tp_group is not None and self.lm_head is not None and self.lm_head.weight.shape[0] != self.cfg.vocab_size:
            from ..ops.lmhead import lmhead_logprob_entropy_tp
            from ..parallel.tensor_parallel import copy_to_tp_region

            return lmhead_logprob_entropy_tp(copy_to_tp_region(hidden, self.tp_group), self.lm_head.weight, labels,
                                             temperature, self.vocab_offset, self.tp_group)
        return ops.lmhead_logprob_entropy(hidden, self.lm_head_weight, labels, temperature)

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return ops.linear(hidden, self.lm_head_weight)

    def values(self, hidden: torch.Tensor) -> torch.Tensor:
        # the value head is a 1-row matrix: a dot product per token (bandwidth-bound, no tensor-core tile)
        return (hidden.float() @ self.score.weight.float().t()).squeeze(-1)

    def forward(self, batch: PackedBatch, labels: Optional[torch.Tensor] = None, temperature: float = 1.0):
        hidden = self.forward_hidden(batch)
        if self.value_head:
            return self.values(hidden)
        if labels is None:
            return self.logits(hidden)
        return self.logprob_entropy(hidden, labels, temperature)


def build_model(cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", value_head: bool = False, seed: int = 0,
                init: bool = True) -> CausalLM:
    m = CausalLM(cfg, dtype=dtype, device=device, value_head=value_head)
    if init:
        m.init_weights(seed)
    return m
