"""Fused lm_head -> token log-prob / entropy without materialising the logits.

Contract of the reference op ``linear_cross_entropy(hidden, weight, labels, temperature)``
(verl/utils/kernel/linear_cross_entropy.py:38-139, kernels.py:563-753):
``logits = hidden @ weight.T / temperature``; returns per-token ``log_softmax(logits)[label]``
and ``entropy(softmax(logits))``, both fp32 ``[T]``.

Forward: one tcgen05 GEMM whose epilogue keeps online-softmax statistics per row.
Backward: per vocab chunk, a second GEMM recomputes the logits tile and emits ``d_logits`` in
bf16, followed by two GEMMs of the same kernel family for ``d_hidden`` and ``d_weight``
(accumulated in fp32). Peak extra memory is ``T x chunk`` bf16 instead of ``T x V`` fp32.
"""

from __future__ import annotations

import torch

from . import _lib
from .gemm import gemm

_DLOGITS_CHUNK = 16384


def _ref_logprob_entropy(hidden, weight, labels, temperature):
    logits = (hidden.float() @ weight.float().t()) / temperature
    lse = torch.logsumexp(logits, dim=-1)
    logp = logits.gather(-1, labels.unsqueeze(-1)).squeeze(-1) - lse
    p = torch.softmax(logits, dim=-1)
    ent = lse - (p * logits).sum(-1)
    return logp, ent


class _LMHeadFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, temperature):
        T, H = hidden.shape
        V = weight.shape[0]
        dev = hidden.device
        splits = _lib.fn("vb_lmhead_num_splits")(T, V)
        scratch = torch.empty(T * splits * 4, dtype=torch.float32, device=dev)
        logp = torch.empty(T, dtype=torch.float32, device=dev)
        ent = torch.empty(T, dtype=torch.float32, device=dev)
        lse = torch.empty(T, dtype=torch.float32, device=dev)
        mean = torch.empty(T, dtype=torch.float32, device=dev)
        rc = _lib.fn("vb_lmhead_logprob_fwd")(
            hidden.data_ptr(), weight.data_ptr(), labels.data_ptr(), T, H, V, 1.0 / temperature,
            scratch.data_ptr(), logp.data_ptr(), ent.data_ptr(), lse.data_ptr(), mean.data_ptr(),
            _lib.status_word(dev).data_ptr(), _lib.stream(),
        )
        _lib.check(rc, "vb_lmhead_logprob_fwd")
        ctx.save_for_backward(hidden, weight, labels, lse, mean)
        ctx.temperature = temperature
        return logp, ent

    @staticmethod
    def backward(ctx, g_logp, g_ent):
        hidden, weight, labels, lse, mean = ctx.saved_tensors
        T, H = hidden.shape
        V = weight.shape[0]
        dev = hidden.device
        g_logp = g_logp.float().contiguous() if g_logp is not None else torch.zeros(T, device=dev)
        g_ent_t = g_ent.float().contiguous() if g_ent is not None else None
        need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        main_grad = getattr(weight, "main_grad", None)
        d_hidden = torch.zeros(T, H, dtype=torch.float32, device=dev) if need_dh else None
        if need_dw:
            d_weight = main_grad if main_grad is not None else torch.zeros(V, H, dtype=torch.float32, device=dev)
        chunk = min(_DLOGITS_CHUNK, V)
        dl = torch.empty(T, chunk, dtype=torch.bfloat16, device=dev)
        fn = _lib.fn("vb_lmhead_dlogits")
        for off in range(0, V, chunk):
            vc = min(chunk, V - off)
            w_chunk = weight[off : off + vc]
            rc = fn(hidden.data_ptr(), w_chunk.data_ptr(), labels.data_ptr(), T, H, vc, off, 1.0 / ctx.temperature,
                    lse.data_ptr(), mean.data_ptr(), g_logp.data_ptr(), _lib.ptr(g_ent_t), dl.data_ptr(), chunk,
                    _lib.status_word(dev).data_ptr(), _lib.stream())
            _lib.check(rc, "vb_lmhead_dlogits")
            dl_v = dl[:, :vc]
            if need_dh:  # dH += dlogits[T,vc] . W[vc,H]
                gemm(dl_v, w_chunk, b_mn=True, out=d_hidden, accumulate=True)
            if need_dw:  # dW[vc,H] += dlogits^T . hidden
                gemm(dl_v, hidden, a_mn=True, b_mn=True, out=d_weight[off : off + vc], accumulate=True)
        dh = d_hidden.to(hidden.dtype) if need_dh else None
        dw = None
        if need_dw and main_grad is None:
            dw = d_weight.to(weight.dtype)
        return dh, dw, None, None


def lmhead_logprob_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                           temperature: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
    """hidden [T,H], weight [V,H], labels [T] int64 -> (logprob [T] fp32, entropy [T] fp32)."""
    if hidden.is_cuda:
        if hidden.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
            raise TypeError("fused lm_head expects bf16 hidden and weight")
        return _LMHeadFn.apply(hidden.contiguous(), weight, labels.contiguous().long(), float(temperature))
    return _ref_logprob_entropy(hidden, weight, labels, temperature)
