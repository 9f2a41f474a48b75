"""Block-scaled fp8 (e4m3): quantisation and GEMM (role of verl/utils/kernel/fp8_kernel.py:53-312 and of the
DeepGEMM / CUTLASS block-fp8 GEMMs that the reference reaches through vLLM, verl/utils/vllm/vllm_fp8_utils.py).

Weights: one fp32 scale per 128 x 128 block; activations: one per (row, 128 columns); ``scale = absmax / 448``, with
``pow2=True`` rounded up to a power of two (UE8M0-representable, the form Blackwell block-scaled kernels consume).
"""

from __future__ import annotations

import torch

from . import _lib

FP8_MAX = 448.0
BLOCK = 128


def _pad16(n: int) -> int:
    return (n + 15) // 16 * 16


def _ceil_pow2(s: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= s (exact: from the exponent, not through log2)."""
    m, e = torch.frexp(s)
    return torch.ldexp(torch.ones_like(s), torch.where(m == 0.5, e - 1, e))


def quantize_weight(w: torch.Tensor, pow2: bool = False):
    """w [N, K] bf16 -> (q [N, K] float8_e4m3fn, scales [ceil(N/128), ceil(K/128)] fp32)."""
    N, K = w.shape
    nb, kb = (N + BLOCK - 1) // BLOCK, (K + BLOCK - 1) // BLOCK
    if w.is_cuda:
        w = w.contiguous()
        q = torch.empty((N, _pad16(K)), dtype=torch.uint8, device=w.device)
        s = torch.empty((nb, kb), dtype=torch.float32, device=w.device)
        rc = _lib.fn("vb_fp8_quant_weight")(w.data_ptr(), w.stride(0), N, K, q.data_ptr(), q.stride(0), s.data_ptr(), int(pow2),
                                            _lib.stream())
        _lib.check(rc, "vb_fp8_quant_weight")
        return q[:, :K].view(torch.float8_e4m3fn), s
    wp = torch.zeros(nb * BLOCK, kb * BLOCK, dtype=torch.float32)
    wp[:N, :K] = w.float()
    blocks = wp.view(nb, BLOCK, kb, BLOCK)
    s = blocks.abs().amax(dim=(1, 3)).clamp(min=1e-10) / FP8_MAX
    if pow2:
        s = _ceil_pow2(s)
    q = (blocks * (1.0 / s)[:, None, :, None]).view(nb * BLOCK, kb * BLOCK)[:N, :K].to(torch.float8_e4m3fn)  # x * (1/s) as the kernel does
    return q, s


def quantize_activation(x: torch.Tensor, pow2: bool = False):
    """x [M, K] bf16 -> (q [M, K] float8_e4m3fn, scales [M, ceil(K/128)] fp32)."""
    M, K = x.shape
    kb = (K + BLOCK - 1) // BLOCK
    if x.is_cuda:
        x = x.contiguous()
        q = torch.empty((M, _pad16(K)), dtype=torch.uint8, device=x.device)
        s = torch.empty((M, kb), dtype=torch.float32, device=x.device)
        rc = _lib.fn("vb_fp8_quant_act")(x.data_ptr(), x.stride(0), M, K, q.data_ptr(), q.stride(0), s.data_ptr(), int(pow2),
                                         _lib.stream())
        _lib.check(rc, "vb_fp8_quant_act")
        return q[:, :K].view(torch.float8_e4m3fn), s
    xp = torch.zeros(M, kb * BLOCK, dtype=torch.float32)
    xp[:, :K] = x.float()
    blocks = xp.view(M, kb, BLOCK)
    s = blocks.abs().amax(-1).clamp(min=1e-10) / FP8_MAX
    if pow2:
        s = _ceil_pow2(s)
    q = (blocks * (1.0 / s)[..., None]).view(M, kb * BLOCK)[:, :K].to(torch.float8_e4m3fn)
    return q, s


def dequantize(q: torch.Tensor, s: torch.Tensor, weight: bool) -> torch.Tensor:
    """fp32 tensor from (q, scales); ``weight`` selects the 128 x 128 (True) or 1 x 128 (False) scale layout."""
    R, K = q.shape
    sk = s.repeat_interleave(BLOCK, dim=1)[:, :K]
    if weight:
        sk = sk.repeat_interleave(BLOCK, dim=0)[:R]
    return q.float() * sk


def fp8_gemm(xq: torch.Tensor, sx: torch.Tensor, wq: torch.Tensor, sw: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 [M, N] = dequant(xq, sx) @ dequant(wq, sw)^T (+ bias)."""
    M, K = xq.shape
    N = wq.shape[0]
    if not xq.is_cuda:
        out = dequantize(xq, sx, False) @ dequantize(wq, sw, True).t()
        return (out + bias.float() if bias is not None else out).to(torch.bfloat16)
    out = torch.empty((M, N), dtype=torch.bfloat16, device=xq.device)
    rc = _lib.fn("vb_fp8_gemm_blockscale")(xq.data_ptr(), wq.data_ptr(), sx.data_ptr(), sw.data_ptr(), out.data_ptr(),
                                           _lib.ptr(bias), M, N, K, xq.stride(0), wq.stride(0), out.stride(0),
                                           _lib.status_word(xq.device).data_ptr(), _lib.stream())
    _lib.check(rc, "vb_fp8_gemm_blockscale")
    return out


def fp8_linear(x: torch.Tensor, wq: torch.Tensor, sw: torch.Tensor, bias: torch.Tensor | None = None, pow2: bool = False):
    """Dynamic activation quantisation + block-scaled GEMM: the rollout-side linear layer on fp8 weights."""
    xq, sx = quantize_activation(x, pow2)
    return fp8_gemm(xq, sx, wq, sw, bias)
