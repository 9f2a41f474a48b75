"""bf16 GEMM on the hand-written tcgen05 kernel, and the Linear autograd function built on it.

Layout convention of :func:`gemm` (C = A . B^T with fp32 accumulation):

* ``a_mn=False``: ``a`` is ``[M, K]`` row-major; ``a_mn=True``: ``a`` is stored ``[K, M]``.
* ``b_mn=False``: ``b`` is ``[N, K]`` row-major; ``b_mn=True``: ``b`` is stored ``[K, N]``.

So a Linear layer needs no transposes: forward ``gemm(x, W)``, data gradient
``gemm(dy, W, b_mn=True)``, weight gradient ``gemm(dy, x, a_mn=True, b_mn=True)``.
CPU tensors take a plain fp32 torch path (used by the CPU test tier only).
"""

from __future__ import annotations

import torch

from . import _lib


def _check_2d(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with unit inner stride, got shape {tuple(t.shape)} stride {t.stride()}")
    if t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        raise ValueError(f"{name}: row stride must be a multiple of 8 elements and the base 16-byte aligned")


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    bias: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype = torch.bfloat16,
    accumulate: bool = False,
) -> torch.Tensor:
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"contraction mismatch: {K} vs {Kb}")
    if not a.is_cuda:
        af = (a.t() if a_mn else a).float()
        bf = (b.t() if b_mn else b).float()
        res = af @ bf.t()
        if bias is not None:
            res = res + bias.float()
        if out is not None:
            if accumulate:
                out += res.to(out.dtype)
            else:
                out.copy_(res)
            return out
        return res.to(out_dtype)
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm expects bf16 operands on CUDA")
    _check_2d(a, "a")
    _check_2d(b, "b")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        accumulate = False
    if out.dtype not in (torch.bfloat16, torch.float32) or out.stride(1) != 1:
        raise TypeError("out must be bf16 or fp32 with unit inner stride")
    if accumulate and out.dtype != torch.float32:
        raise TypeError("accumulate requires an fp32 output")
    stream = _lib.stream()
    ws, counters = _splitk_workspace(a.device, stream) if M <= _SPLITK_MAX_M else (None, None)
    rc = _lib.fn("vb_gemm_bf16_ws")(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), _lib.ptr(bias), M, N, K,
        a.stride(0), b.stride(0), out.stride(0), int(a_mn), int(b_mn),
        int(out.dtype == torch.float32), int(accumulate),
        _lib.ptr(ws), ws.numel() * 4 if ws is not None else 0, _lib.ptr(counters), _SPLITK_COUNTERS if ws is not None else 0,
        _lib.status_word(a.device).data_ptr(), stream,
    )
    _lib.check(rc, "vb_gemm_bf16")
    return out


# Split-K scratch for skinny problems (decode-time projections). One workspace per (device, stream): calls that
# share one are ordered by the stream. Launches recorded under graph capture share one more workspace per device
# (created by the first eager call, kept for the life of the process so that replays find it): graphs that
# contain split-K GEMMs must therefore not be replayed concurrently with each other.
_SPLITK_MAX_M = 256
_SPLITK_BYTES = 32 << 20
_SPLITK_COUNTERS = 4096
_splitk_ws: dict = {}


def _splitk_workspace(device, stream):
    capturing = torch.cuda.is_current_stream_capturing()
    key = (device.index, "capture" if capturing else stream)
    got = _splitk_ws.get(key)
    if got is None:
        if capturing:
            # allocating under capture would put the buffers in the graph's private pool
            return None, None
        for k in (key, (device.index, "capture")):
            if k not in _splitk_ws:
                _splitk_ws[k] = (torch.empty(_SPLITK_BYTES // 4, dtype=torch.float32, device=device),
                                 torch.zeros(_SPLITK_COUNTERS, dtype=torch.int32, device=device))
        got = _splitk_ws[key]
    return got


class _LinearFn(torch.autograd.Function):
    """y = x W^T (+ b). If ``weight.main_grad`` exists (fp32, same shape) the weight gradient
    is accumulated into it by the GEMM epilogue and autograd sees ``None`` for the weight."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        x2 = x if x.dim() == 2 else x.reshape(-1, x.shape[-1])
        y = gemm(x2, weight, bias=bias, out_dtype=x.dtype)
        # a 2-D input returns the freshly allocated result itself (not a view), so callers may update it in place
        return y if x.dim() == 2 else y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True, out_dtype=x.dtype).reshape(x.shape)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main_grad, accumulate=True)
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    return _LinearFn.apply(x, weight, bias)
