"""Vision side of the Qwen2-VL / Qwen2.5-VL / Qwen3-VL families: ViT tower with 2-D rotary attention and the 2 x 2 patch
merger, multimodal RoPE position ids, and the merge of image embeddings into the token stream.

The reference takes these models from ``transformers`` and patches their forward for packed inputs and mrope
(verl/models/transformers/qwen2_vl.py:1-548; position ids: ``get_rope_index`` there and
verl/utils/tensordict_utils.py:847). Here the tower runs on the same native linear / attention ops as the decoder
(packed patches, one attention segment per frame).
"""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops


@dataclass
class VisionConfig:
    depth: int = 32
    embed_dim: int = 1280
    hidden_size: int = 3584          # width of the language model the merger projects to
    num_heads: int = 16
    mlp_ratio: float = 4.0
    in_channels: int = 3
    patch_size: int = 14
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    hidden_act: str = "quick_gelu"
    # Qwen2.5-VL: RMSNorm instead of LayerNorm, gated SiLU MLP of ``intermediate_size``, attention inside windows of
    # ``window_size`` pixels except in the blocks ``fullatt_block_indexes`` (verl/models/transformers/qwen2_vl.py serves
    # both generations through transformers; here ``variant`` selects the block layout)
    variant: str = "qwen2_vl"
    intermediate_size: int = 0
    window_size: int = 112
    fullatt_block_indexes: tuple = (7, 15, 23, 31)
    # Qwen3-VL (verl/models/transformers/qwen3_vl.py): LayerNorm blocks with a two-matrix tanh-GELU MLP and full
    # attention, a learned position table of ``num_position_embeddings`` entries (a square grid, interpolated to the
    # image's patch grid) added to the patch embeddings, and "deepstack" mergers that read the hidden states after the
    # blocks ``deepstack_visual_indexes``; their outputs are added to the language model's hidden states
    num_position_embeddings: int = 2304
    deepstack_visual_indexes: tuple = ()

    @classmethod
    def from_dict(cls, d: dict) -> "VisionConfig":
        d = dict(d)
        if "deepstack_visual_indexes" in d or d.get("variant") == "qwen3_vl":
            if "out_hidden_size" in d:
                d["embed_dim"], d["hidden_size"] = d["hidden_size"], d.pop("out_hidden_size")
            d["variant"] = "qwen3_vl"
            d["deepstack_visual_indexes"] = tuple(d.get("deepstack_visual_indexes") or ())
            d.setdefault("hidden_act", "gelu_pytorch_tanh")
        elif "out_hidden_size" in d or d.get("variant") == "qwen2_5_vl":
            # the HF Qwen2.5-VL vision config calls the tower's width ``hidden_size`` and the language model's width
            # ``out_hidden_size``
            if "out_hidden_size" in d:
                d["embed_dim"], d["hidden_size"] = d["hidden_size"], d["out_hidden_size"]
            d["variant"] = "qwen2_5_vl"
            d.setdefault("hidden_act", "silu")
        if "in_chans" in d and "in_channels" not in d:
            d["in_channels"] = d["in_chans"]
        if "fullatt_block_indexes" in d:
            d["fullatt_block_indexes"] = tuple(d["fullatt_block_indexes"])
        known = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in d.items() if k in known})

    def to_dict(self) -> dict:
        return asdict(self)

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size


class _Lin(nn.Module):
    """Linear with bias on the native GEMM (CPU: torch)."""

    def __init__(self, i: int, o: int, bias: bool, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(o, i, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(o, dtype=dtype, device=device)) if bias else None

    def forward(self, x):
        if x.is_cuda and x.shape[-1] % 8 == 0 and self.weight.shape[0] % 8 == 0:
            return ops.linear(x, self.weight, self.bias)
        return F.linear(x, self.weight, self.bias)


class _LayerNormW(nn.Module):
    def __init__(self, dim: int, dtype, device, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device))
        self.eps = eps

    def forward(self, x):
        return F.layer_norm(x.float(), (x.shape[-1],), self.weight.float(), self.bias.float(), self.eps).to(x.dtype)


class _RMSNormW(nn.Module):
    def __init__(self, dim: int, dtype, device, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.eps = eps

    def forward(self, x):
        h = x.float()
        return (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()).to(x.dtype)


def _rotate_half(x):
    a, b = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2 :]
    return torch.cat([-b, a], -1)


class VisionBlock(nn.Module):
    def __init__(self, c: VisionConfig, dtype, device):
        super().__init__()
        self.c = c
        Norm = _RMSNormW if c.variant == "qwen2_5_vl" else _LayerNormW
        self.norm1 = Norm(c.embed_dim, dtype, device)
        self.norm2 = Norm(c.embed_dim, dtype, device)
        self.qkv = _Lin(c.embed_dim, 3 * c.embed_dim, True, dtype, device)
        self.proj = _Lin(c.embed_dim, c.embed_dim, True, dtype, device)
        if c.variant == "qwen2_5_vl":
            hid = int(c.intermediate_size)
            self.fc_gate = _Lin(c.embed_dim, hid, True, dtype, device)
            self.fc_up = _Lin(c.embed_dim, hid, True, dtype, device)
            self.fc1 = None
        else:
            hid = int(c.intermediate_size) if c.variant == "qwen3_vl" else int(c.embed_dim * c.mlp_ratio)
            self.fc1 = _Lin(c.embed_dim, hid, True, dtype, device)
        self.fc2 = _Lin(hid, c.embed_dim, True, dtype, device)

    def forward(self, x, cu_seqlens, max_seqlen, cos, sin):
        c = self.c
        N = x.shape[0]
        hd = c.embed_dim // c.num_heads
        qkv = self.qkv(self.norm1(x)).view(N, 3, c.num_heads, hd)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
        q = (q.float() * cos + _rotate_half(q.float()) * sin).to(x.dtype)
        k = (k.float() * cos + _rotate_half(k.float()) * sin).to(x.dtype)
        a = ops.attention_varlen(q.contiguous(), k.contiguous(), v.contiguous(), cu_seqlens, max_seqlen, causal=False)
        x = x + self.proj(a.reshape(N, c.embed_dim))
        y = self.norm2(x)
        if self.fc1 is None:  # gated SiLU
            h = F.silu(self.fc_gate(y)) * self.fc_up(y)
        else:
            h = self.fc1(y)
            if c.hidden_act == "quick_gelu":
                h = h * torch.sigmoid(1.702 * h)
            else:
                h = F.gelu(h, approximate="tanh" if c.hidden_act == "gelu_pytorch_tanh" else "none")
        return x + self.fc2(h)


class _DeepstackMerger(nn.Module):
    """Merger of a deepstack tap: LayerNorm over the concatenated 2 x 2 unit, two linears with a GELU between."""

    def __init__(self, c: VisionConfig, dtype, device):
        super().__init__()
        wide = c.embed_dim * c.spatial_merge_size ** 2
        self.norm = _LayerNormW(wide, dtype, device)
        self.fc1 = _Lin(wide, wide, True, dtype, device)
        self.fc2 = _Lin(wide, c.hidden_size, True, dtype, device)

    def forward(self, x):
        return self.fc2(F.gelu(self.fc1(self.norm(x.view(-1, self.norm.weight.shape[0])))))


class VisionTower(nn.Module):
    """``pixel_values [N, C * T * P * P]`` (patches already in 2 x 2 merge order) + ``grid_thw [n_images, 3]`` ->
    ``[N / merge^2, hidden_size]`` embeddings, one per image placeholder token."""

    def __init__(self, c: VisionConfig, dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        self.c = c
        # the Conv3d of the reference, as a GEMM
        self.patch_embed = _Lin(c.patch_dim, c.embed_dim, c.variant == "qwen3_vl", dtype, device)
        self.blocks = nn.ModuleList([VisionBlock(c, dtype, device) for _ in range(c.depth)])
        self.ln_q = (_RMSNormW if c.variant == "qwen2_5_vl" else _LayerNormW)(c.embed_dim, dtype, device)
        m2 = c.spatial_merge_size ** 2
        self.merge_fc1 = _Lin(c.embed_dim * m2, c.embed_dim * m2, True, dtype, device)
        self.merge_fc2 = _Lin(c.embed_dim * m2, c.hidden_size, True, dtype, device)
        self.pos_embed = self.deepstack = None
        if c.variant == "qwen3_vl":
            self.pos_embed = nn.Embedding(c.num_position_embeddings, c.embed_dim, dtype=dtype, device=device)
            self.deepstack = nn.ModuleList([_DeepstackMerger(c, dtype, device) for _ in c.deepstack_visual_indexes])

    @property
    def num_deepstack(self) -> int:
        return len(self.deepstack) if self.deepstack is not None else 0

    def interpolated_pos_embed(self, grid_thw: torch.Tensor) -> torch.Tensor:
        """Qwen3-VL: bilinear interpolation of the learned ``side x side`` position table to every image's ``h x w``
        patch grid (corners aligned), repeated for every frame, in the merge-block order of the patches."""
        c = self.c
        side = int(c.num_position_embeddings ** 0.5)
        m = c.spatial_merge_size
        table = self.pos_embed.weight
        out = []
        for t, h, w in grid_thw.tolist():
            ys = torch.linspace(0, side - 1, h, device=table.device)
            xs = torch.linspace(0, side - 1, w, device=table.device)
            y0, x0 = ys.long(), xs.long()
            y1, x1 = (y0 + 1).clamp(max=side - 1), (x0 + 1).clamp(max=side - 1)
            dy, dx = (ys - y0).to(table.dtype), (xs - x0).to(table.dtype)
            pick = lambda yy, xx: table[(yy[:, None] * side + xx[None, :]).reshape(-1)].view(h, w, -1)  # noqa: E731
            wy0, wy1, wx0, wx1 = (1 - dy)[:, None, None], dy[:, None, None], (1 - dx)[None, :, None], dx[None, :, None]
            pe = pick(y0, x0) * wy0 * wx0 + pick(y0, x1) * wy0 * wx1 + pick(y1, x0) * wy1 * wx0 + pick(y1, x1) * wy1 * wx1
            pe = pe.view(h // m, m, w // m, m, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)
            out.append(pe.repeat(t, 1))
        return torch.cat(out, 0)

    def init_weights(self, seed: int = 0):
        g = torch.Generator(device=self.patch_embed.weight.device)
        g.manual_seed(seed)
        with torch.no_grad():
            for n, p in self.named_parameters():
                if n.endswith("weight") and p.dim() == 2:
                    p.copy_(torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0.0, 0.02, generator=g))
        return self

    def rot_pos(self, grid_thw: torch.Tensor):
        """(cos, sin) [N, 1, head_dim] of the 2-D rotary embedding: half of the frequencies follow the patch's row,
        half its column, in the merge-block order of the patches."""
        c = self.c
        m = c.spatial_merge_size
        hd = c.embed_dim // c.num_heads
        dim = hd // 2
        dev = grid_thw.device
        ids = []
        for t, h, w in grid_thw.tolist():
            hp = torch.arange(h, device=dev).unsqueeze(1).expand(-1, w)
            wp = torch.arange(w, device=dev).unsqueeze(0).expand(h, -1)
            hp = hp.reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            wp = wp.reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            ids.append(torch.stack([hp, wp], -1).repeat(t, 1))
        ids = torch.cat(ids, 0)
        inv = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float32, device=dev) / dim))
        freqs = torch.arange(int(grid_thw[:, 1:].max()), dtype=torch.float32, device=dev)[:, None] * inv[None]
        emb = freqs[ids].flatten(1)                    # [N, dim]: row frequencies, then column frequencies
        emb = torch.cat([emb, emb], -1)                # [N, head_dim]
        return emb.cos()[:, None, :], emb.sin()[:, None, :]

    def window_order(self, grid_thw: torch.Tensor):
        """Qwen2.5-VL: (order of the merged-patch units window by window, window boundaries in patches). The merged grid
        of every frame is cut into squares of ``window_size / patch_size / merge`` units; a unit list per window, frame by
        frame, image by image; windows at the right / bottom edge are smaller."""
        c = self.c
        ws = c.window_size // c.spatial_merge_size // c.patch_size
        m2 = c.spatial_merge_size ** 2
        order, bounds, base = [], [0], 0
        for t, h, w in grid_thw.tolist():
            gh, gw = h // c.spatial_merge_size, w // c.spatial_merge_size
            unit = torch.arange(t * gh * gw).view(t, gh, gw)
            for f in range(t):
                for r0 in range(0, gh, ws):
                    for c0 in range(0, gw, ws):
                        win = unit[f, r0 : r0 + ws, c0 : c0 + ws].reshape(-1)
                        order.append(win + base)
                        bounds.append(bounds[-1] + win.numel() * m2)
            base += t * gh * gw
        return torch.cat(order), torch.tensor(bounds, dtype=torch.int32)

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor, return_deepstack: bool = False):
        """``return_deepstack`` (Qwen3-VL): also the list of deepstack features, each ``[N / merge^2, hidden_size]``."""
        c = self.c
        x = self.patch_embed(pixel_values.to(self.patch_embed.weight.dtype))
        if self.pos_embed is not None:
            x = x + self.interpolated_pos_embed(grid_thw).to(x.dtype)
        cos, sin = self.rot_pos(grid_thw)
        per_frame = (grid_thw[:, 1] * grid_thw[:, 2]).repeat_interleave(grid_thw[:, 0])
        cu = F.pad(per_frame.cumsum(0), (1, 0)).to(torch.int32)
        max_len = int(per_frame.max())
        m2 = c.spatial_merge_size ** 2
        if c.variant == "qwen2_5_vl":
            # patches travel window by window (whole merge units stay together); the merged outputs go back to the
            # original order at the end
            order, cu_win = self.window_order(grid_thw.cpu())
            order, cu_win = order.to(x.device), cu_win.to(x.device)
            max_win = int((cu_win[1:] - cu_win[:-1]).max())
            regroup = lambda t: t.reshape(t.shape[0] // m2, m2, *t.shape[1:])[order].reshape(t.shape)  # noqa: E731
            x, cos, sin = regroup(x), regroup(cos), regroup(sin)
            for i, blk in enumerate(self.blocks):
                full = i in c.fullatt_block_indexes
                x = blk(x, cu if full else cu_win, max_len if full else max_win, cos, sin)
            x = self.ln_q(x).view(-1, c.embed_dim * m2)
            out = self.merge_fc2(F.gelu(self.merge_fc1(x)))
            return out[torch.argsort(order)]
        taps = []
        for i, blk in enumerate(self.blocks):
            x = blk(x, cu, max_len, cos, sin)
            if self.deepstack is not None and i in c.deepstack_visual_indexes:
                taps.append(self.deepstack[c.deepstack_visual_indexes.index(i)](x))
        x = self.ln_q(x).view(-1, c.embed_dim * m2)
        out = self.merge_fc2(F.gelu(self.merge_fc1(x)))
        return (out, taps) if return_deepstack else out


def get_rope_index(input_ids: torch.Tensor, image_grid_thw: Optional[torch.Tensor], image_token_id: int,
                   spatial_merge_size: int = 2, video_grid_thw: Optional[torch.Tensor] = None,
                   video_token_id: Optional[int] = None, split_video_frames: bool = False) -> tuple[torch.Tensor, int]:
    """Multimodal RoPE positions of ONE sequence of token ids (no padding): ``[3, L]`` (temporal, height, width) and
    the delta to add to a text position after the sequence (``max position + 1 - L``). Text tokens advance all three
    axes together; the placeholder tokens of an image take (frame, row, column) of their merged patch, offset by the
    position at which the image starts; the text after it continues from the largest position so far + 1."""
    L = input_ids.numel()
    dev = input_ids.device
    ids = input_ids.tolist()
    grids = []
    if image_grid_thw is not None:
        grids += [(image_token_id, g) for g in image_grid_thw.tolist()]
    vids = [(video_token_id, g) for g in video_grid_thw.tolist()] if video_grid_thw is not None else []
    if split_video_frames:
        # Qwen3-VL: timestamps separate the frames of a video in the prompt, so every frame is a grid of its own
        vids = [(tok, [1, h, w]) for tok, (t, h, w) in vids for _ in range(t)]
    if not grids and not vids:
        p = torch.arange(L, device=dev)
        return torch.stack([p, p, p]), 0
    out = []
    st, nxt = 0, 0
    img_it, vid_it = iter(grids), iter(vids)
    while st < L:
        ends = [ids.index(tok, st) if tok is not None and tok in ids[st:] else L + 1 for tok in (image_token_id, video_token_id)]
        if min(ends) > L:
            break
        use_img = ends[0] <= ends[1]
        ed = ends[0] if use_img else ends[1]
        nxt_grid = next(img_it if use_img else vid_it, None)
        if nxt_grid is None:
            # more placeholder ids than grids: a policy sampled the placeholder id as an ordinary token (a generated
            # response); everything from here on is text
            break
        _, (t, h, w) = nxt_grid
        gh, gw = h // spatial_merge_size, w // spatial_merge_size
        n_text = ed - st
        if n_text:
            p = torch.arange(n_text, device=dev) + nxt
            out.append(torch.stack([p, p, p]))
            nxt += n_text
        ti = torch.arange(t, device=dev).view(-1, 1).expand(-1, gh * gw).flatten()
        hi = torch.arange(gh, device=dev).view(1, -1, 1).expand(t, -1, gw).flatten()
        wi = torch.arange(gw, device=dev).view(1, 1, -1).expand(t, gh, -1).flatten()
        out.append(torch.stack([ti, hi, wi]) + nxt)
        nxt = int(out[-1].max()) + 1
        st = ed + t * gh * gw
    if st < L:
        p = torch.arange(L - st, device=dev) + nxt
        out.append(torch.stack([p, p, p]))
    pos = torch.cat(out, 1)
    return pos, int(pos.max()) + 1 - L
