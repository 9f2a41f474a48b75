"""Mixture-of-experts building blocks: device-side routing layout and grouped GEMMs (one launch for all experts).

The routed tokens are sorted by expert into a buffer in which every expert's rows are padded to a multiple of 128,
so that a GEMM tile never straddles two experts; ``blk_expert`` names the expert of every 128-row block. Nothing is
read back to the host (no per-expert Python loop, no ``.tolist()``): the padded size is the static upper bound
``T * k + E * 127``. The reference leaves this to Megatron / vLLM fused-MoE kernels (grouped GEMM + permute).
"""

from __future__ import annotations

import torch

from . import _lib

BLK = 128


def moe_layout(top_i: torch.Tensor, E: int):
    """top_i [T, k] expert ids -> (dest [T*k] row of every (token, slot) pair in the padded sorted buffer,
    blk_expert int32 [P / 128], expert_off int32 [E + 1] padded row offsets, P)."""
    T, k = top_i.shape
    flat = top_i.reshape(-1)
    P = ((T * k + E * (BLK - 1)) + BLK - 1) // BLK * BLK
    order = torch.argsort(flat, stable=True)
    # (torch.bincount would read its maximum back to the host: not capturable in a CUDA graph)
    counts = torch.zeros(E, dtype=torch.long, device=flat.device).scatter_add_(0, flat, torch.ones_like(flat))
    padded = (counts + BLK - 1) // BLK * BLK
    zero = torch.zeros(1, dtype=counts.dtype, device=counts.device)
    start = torch.cat([zero, counts.cumsum(0)])          # unpadded offsets
    off = torch.cat([zero, padded.cumsum(0)])            # padded offsets
    e_sorted = flat[order]
    rank_in_e = torch.arange(T * k, device=flat.device) - start[e_sorted]
    dest_sorted = off[e_sorted] + rank_in_e
    dest = torch.empty_like(dest_sorted)
    dest[order] = dest_sorted
    blk_start = torch.arange(0, P, BLK, device=flat.device)
    blk_expert = torch.searchsorted(off[1:].contiguous(), blk_start, right=True)
    blk_expert = torch.where(blk_start < off[-1], blk_expert, torch.full_like(blk_expert, -1)).to(torch.int32)
    return dest, blk_expert, off.to(torch.int32), P


def _grouped(a, b, c, M, N, K, a_mn, b_mn, accumulate, mode, E, blk_expert, expert_off):
    rc = _lib.fn("vb_grouped_gemm_bf16")(a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, a.stride(0), b.stride(-2),
                                         c.stride(-2), int(a_mn), int(b_mn), int(c.dtype == torch.float32), int(accumulate),
                                         mode, E, _lib.ptr(blk_expert), _lib.ptr(expert_off),
                                         _lib.status_word(a.device).data_ptr(), _lib.stream())
    _lib.check(rc, "vb_grouped_gemm_bf16")


class _GroupedLinearFn(torch.autograd.Function):
    """y[rows of e] = xs[rows of e] @ W[e]^T for all experts at once. W [E, N, K]."""

    @staticmethod
    def forward(ctx, xs, weight, blk_expert, expert_off):
        E, N, K = weight.shape
        P = xs.shape[0]
        y = torch.zeros((P, N), dtype=xs.dtype, device=xs.device)  # unused blocks stay zero
        _grouped(xs, weight, y, P, N, K, False, False, False, 1, E, blk_expert, None)
        ctx.save_for_backward(xs, weight, blk_expert, expert_off)
        return y

    @staticmethod
    def backward(ctx, dy):
        xs, weight, blk_expert, expert_off = ctx.saved_tensors
        E, N, K = weight.shape
        P = xs.shape[0]
        dy = dy.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.zeros((P, K), dtype=xs.dtype, device=xs.device)
            # dX = dY . W[e]: W[e] [N, K] is the MN-major B operand (stored [contraction, out])
            _grouped(dy, weight, dx, P, K, N, False, True, False, 1, E, blk_expert, None)
        dw = None
        if ctx.needs_input_grad[1]:
            main = getattr(weight, "main_grad", None)
            acc = main if main is not None else torch.zeros((E, N, K), dtype=torch.float32, device=xs.device)
            # dW[e] += dY_e^T . X_e, contraction over the expert's (zero-padded) rows
            _grouped(dy, xs, acc, N, K, P, True, True, True, 2, E, None, expert_off)
            dw = None if main is not None else acc.to(weight.dtype)
        return dx, dw, None, None


def grouped_linear(xs: torch.Tensor, weight: torch.Tensor, blk_expert: torch.Tensor, expert_off: torch.Tensor) -> torch.Tensor:
    if not xs.is_cuda:
        E = weight.shape[0]
        y = torch.zeros(xs.shape[0], weight.shape[1], dtype=xs.dtype, device=xs.device)
        off = expert_off.tolist()
        for e in range(E):
            if off[e + 1] > off[e]:
                y[off[e] : off[e + 1]] = xs[off[e] : off[e + 1]] @ weight[e].t()
        return y
    return _GroupedLinearFn.apply(xs, weight, blk_expert, expert_off)


def moe_mlp(x: torch.Tensor, top_i: torch.Tensor, top_w: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, swiglu,
            expert_offset: int = 0, num_experts: int | None = None):
    """Routed expert MLP. x [T, H], top_i / top_w [T, k], gate_up [E, 2I, H], down [E, H, I].

    Expert parallelism over replicated tokens: with ``num_experts`` larger than ``E`` the matrices are the experts
    ``[expert_offset, expert_offset + E)`` of the layer; pairs routed elsewhere fall into a spare bucket whose blocks
    the grouped GEMM skips, and the result is this rank's partial sum (the ranks' results add up to the layer's)."""
    T, H = x.shape
    k = top_i.shape[1]
    E = gate_up.shape[0]
    if num_experts is not None and num_experts != E:
        local = top_i - expert_offset
        local = torch.where((local >= 0) & (local < E), local, torch.full_like(local, E))
        dest, blk_expert, expert_off, P = moe_layout(local, E + 1)
        blk_expert = torch.where(blk_expert == E, torch.full_like(blk_expert, -1), blk_expert)
        top_w = torch.where(local < E, top_w, torch.zeros_like(top_w))
        expert_off = expert_off[: E + 1].contiguous()
    else:
        dest, blk_expert, expert_off, P = moe_layout(top_i, E)
    tok = torch.arange(T * k, device=x.device) // k
    xs = torch.zeros((P, H), dtype=x.dtype, device=x.device).index_copy(0, dest, x.index_select(0, tok))
    h = swiglu(grouped_linear(xs, gate_up, blk_expert, expert_off))
    out = grouped_linear(h, down, blk_expert, expert_off)
    picked = out.index_select(0, dest).view(T, k, H)
    return (picked * top_w.to(x.dtype).unsqueeze(-1)).sum(1)
