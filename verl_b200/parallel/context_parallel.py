"""Context parallelism: every rank holds two zig-zag chunks of every sequence and attends to the gathered keys.

The reference reaches context parallelism only through Megatron / TransformerEngine: ``preprocess_packed_seqs``
(verl/models/mcore/util.py:25-116) pads every sequence to a multiple of ``2 * cp`` and gives rank r the chunks r and
``2 * cp - 1 - r`` of it (the zig-zag split balances causal attention work), TransformerEngine's ring attention does
the rest, and ``postprocess_packed_seqs`` (:118-160) gathers the outputs back. Here:

* :func:`cp_local_index` — which tokens of the packed stream a rank holds, chunk-major (first every sequence's low
  chunk, then every sequence's high chunk), so that "chunk a of all sequences" is one packed varlen batch;
* keys and values of all ranks are all-gathered (their gradient comes back by reduce-scatter); for a query chunk a the
  attention over the key chunks 0..a is computed chunk pair by chunk pair with the ordinary varlen kernels (chunk a
  against itself causally, against every earlier chunk in full) and merged through the log-sum-exp of each part;
* the backward runs the flash-attention backward of every chunk pair with the MERGED output and the GLOBAL
  log-sum-exp, which yields exactly that pair's share of dQ, dK and dV (the identity behind ring attention), so no
  gradient of a log-sum-exp is ever needed.

Work per rank: ``2 * cp + 1`` chunk pairs, the same on every rank.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


# --------------------------------------------------------------------------------------------------- layout
def cp_chunk_lens(cu_seqlens: torch.Tensor, cp: int) -> torch.Tensor:
    """Length of one chunk of every sequence: ``ceil(len / (2 * cp))``."""
    lens = (cu_seqlens[1:] - cu_seqlens[:-1]).long()
    return (lens + 2 * cp - 1) // (2 * cp)


def cp_local_index(cu_seqlens: torch.Tensor, cp_rank: int, cp: int):
    """Indices into the packed stream of the tokens that rank ``cp_rank`` holds, in chunk-major order, ``-1`` where the
    rank holds padding (a sequence is padded at its END to a multiple of ``2 * cp``). Returns ``(idx [2 * Tc],
    cu_chunk int32 [B + 1], offs [2 * Tc])``: ``offs`` is the position of every local token inside its (padded)
    sequence, ``Tc = sum of chunk lengths``."""
    cu = cu_seqlens.long().cpu()
    lens = cu[1:] - cu[:-1]
    c = (lens + 2 * cp - 1) // (2 * cp)
    cu_chunk = torch.zeros(c.numel() + 1, dtype=torch.int32)
    cu_chunk[1:] = torch.cumsum(c, 0)
    idx_parts, off_parts = [], []
    for chunk in (cp_rank, 2 * cp - 1 - cp_rank):
        for s in range(lens.numel()):
            o = torch.arange(int(c[s])) + chunk * int(c[s])
            off_parts.append(o)
            idx_parts.append(torch.where(o < lens[s], o + cu[s], torch.full_like(o, -1)))
    dev = cu_seqlens.device
    return torch.cat(idx_parts).to(dev), cu_chunk.to(dev), torch.cat(off_parts).to(dev)


# --------------------------------------------------------------------------------------------------- collectives
class _AllGatherCat(torch.autograd.Function):
    """[n, ...] on every rank -> [world * n, ...] (rank-major). Backward: reduce-scatter (sum) of the gradient."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = dist.get_world_size(group)
        out = torch.empty((w * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        w = dist.get_world_size(ctx.group)
        g = g.contiguous()
        out = torch.empty((g.shape[0] // w,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        if g.is_cuda:
            dist.reduce_scatter_tensor(out, g, group=ctx.group)
        else:  # gloo has no reduce-scatter: all-reduce and keep this rank's part
            dist.all_reduce(g, group=ctx.group)
            r = dist.get_rank(ctx.group)
            out = g[r * out.shape[0] : (r + 1) * out.shape[0]].clone()
        return out, None


# --------------------------------------------------------------------------------------------------- attention
def _ref_block(q, k, v, cu, causal: bool, scale: float):
    """(out fp32 [T, Hq, D], lse fp32 [Hq, T]) of one chunk pair in plain torch ops (differentiable; the CPU path)."""
    G = q.shape[1] // k.shape[1]
    outs, lses = [], []
    b = cu.tolist()
    for s, e in zip(b[:-1], b[1:]):
        qs = q[s:e].float().transpose(0, 1)
        ks = k[s:e].float().repeat_interleave(G, dim=1).transpose(0, 1)
        vs = v[s:e].float().repeat_interleave(G, dim=1).transpose(0, 1)
        sc = qs @ ks.transpose(1, 2) * scale
        if causal:
            n = e - s
            sc = sc.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool, device=q.device), 1), float("-inf"))
        lse = torch.logsumexp(sc, -1)
        outs.append((torch.softmax(sc, -1) @ vs).transpose(0, 1))
        lses.append(lse)
    return torch.cat(outs, 0), torch.cat(lses, 1)


def _pairs(cp_rank: int, cp: int):
    """(local query chunk 0 / 1, global key chunk, causal) of every chunk pair this rank computes."""
    out = []
    for qi, a in enumerate((cp_rank, 2 * cp - 1 - cp_rank)):
        for b in range(a + 1):
            out.append((qi, b, b == a))
    return out


def _merge(parts):
    """[(out [T, Hq, D], lse [Hq, T])] -> merged (out fp32, lse fp32)."""
    lse = torch.logsumexp(torch.stack([l for _, l in parts]), 0)
    out = sum(o.float() * torch.exp(l - lse).transpose(0, 1).unsqueeze(-1) for o, l in parts)
    return out, lse


class _CPAttnKernelFn(torch.autograd.Function):
    """Chunk-pair attention on the tcgen05 kernels. q [2 * Tc, Hq, 128] (two local chunks, chunk-major), k / v
    [2 * cp * Tc, Hk, 128] (all chunks in GLOBAL chunk order)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_chunk, max_chunk, cp_rank, cp, scale):
        from ..ops.attention import flash_fwd

        Tc = q.shape[0] // 2
        outs, lses = [], []
        for qi in range(2):
            parts = []
            for pqi, b, causal in _pairs(cp_rank, cp):
                if pqi != qi:
                    continue
                parts.append(flash_fwd(q[qi * Tc : (qi + 1) * Tc], k[b * Tc : (b + 1) * Tc], v[b * Tc : (b + 1) * Tc], cu_chunk,
                                       max_chunk, causal, scale, need_lse=True))
            o, l = _merge(parts)
            outs.append(o.to(q.dtype))
            lses.append(l)
        out = torch.cat(outs, 0)
        ctx.save_for_backward(q, k, v, out, lses[0], lses[1], cu_chunk)
        ctx.meta = (max_chunk, cp_rank, cp, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..ops.attention import flash_bwd

        q, k, v, out, lse0, lse1, cu_chunk = ctx.saved_tensors
        max_chunk, cp_rank, cp, scale = ctx.meta
        Tc = q.shape[0] // 2
        dout = dout.contiguous()
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        dk = torch.zeros(k.shape, dtype=torch.float32, device=k.device)
        dv = torch.zeros(v.shape, dtype=torch.float32, device=v.device)
        for qi, b, causal in _pairs(cp_rank, cp):
            qs, ks = slice(qi * Tc, (qi + 1) * Tc), slice(b * Tc, (b + 1) * Tc)
            # merged output + global log-sum-exp: the kernel's P = exp(S - lse) is then this pair's share of the
            # global softmax, and delta = rowsum(dout * out) is the global one
            gq, gk, gv = flash_bwd(q[qs], k[ks], v[ks], out[qs], (lse0, lse1)[qi], dout[qs], cu_chunk, max_chunk, causal, scale)
            dq[qs] += gq.float()
            dk[ks] += gk.float()
            dv[ks] += gv.float()
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None, None, None, None


def cp_attention_local(q, k_all, v_all, cu_chunk, max_chunk: int, cp_rank: int, cp: int, scale: Optional[float] = None):
    """Causal attention of this rank's two query chunks over the gathered keys / values (global chunk order)."""
    D = q.shape[-1]
    scale = scale if scale is not None else D ** -0.5
    from ..ops.attention import _native_fwd_ok

    if q.is_cuda and _native_fwd_ok(q, k_all, v_all):
        return _CPAttnKernelFn.apply(q, k_all, v_all, cu_chunk, int(max_chunk), int(cp_rank), int(cp), float(scale))
    Tc = q.shape[0] // 2
    outs = []
    for qi in range(2):
        parts = [_ref_block(q[qi * Tc : (qi + 1) * Tc], k_all[b * Tc : (b + 1) * Tc], v_all[b * Tc : (b + 1) * Tc], cu_chunk, causal, scale)
                 for pqi, b, causal in _pairs(cp_rank, cp) if pqi == qi]
        outs.append(_merge(parts)[0].to(q.dtype))
    return torch.cat(outs, 0)


def to_global_chunk_order(x_gathered: torch.Tensor, cp: int) -> torch.Tensor:
    """Rank-major gathered chunks ``[rank 0: chunk 0, chunk 2cp-1 | rank 1: chunk 1, chunk 2cp-2 | ...]`` -> chunks in
    the order 0 .. 2cp-1."""
    Tc = x_gathered.shape[0] // (2 * cp)
    parts = x_gathered.view(cp, 2, Tc, *x_gathered.shape[1:])
    order = [None] * (2 * cp)
    for r in range(cp):
        order[r] = parts[r, 0]
        order[2 * cp - 1 - r] = parts[r, 1]
    return torch.cat(order, 0)


def cp_attention(q, k, v, cu_chunk, max_chunk: int, group, scale: Optional[float] = None):
    """q / k / v: this rank's two chunks (chunk-major). Gathers keys and values over ``group`` and attends."""
    cp, r = dist.get_world_size(group), dist.get_rank(group)
    k_all = to_global_chunk_order(_AllGatherCat.apply(k, group), cp)
    v_all = to_global_chunk_order(_AllGatherCat.apply(v, group), cp)
    return cp_attention_local(q, k_all, v_all, cu_chunk, max_chunk, r, cp, scale)
