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


# ---------------------------------------------------------------------------------------------------------------
# Vocabulary-parallel variant: every rank of a tensor-parallel group holds V / tp rows of the lm_head. The per-shard
# online-softmax statistics are merged across the group (role of verl/utils/kernel/kernels.py:438-557 with its
# all-reduces at :702-734):
#     lse = log sum_r exp(lse_r)            label logit = sum_r [label in shard r] logit_r
#     E_p[logit] = sum_r exp(lse_r - lse) E_{p_r}[logit]
# The backward recomputes the local logits tile by tile against the GLOBAL lse / mean (the same d_logits kernel), so
# d_weight is local and d_hidden is this rank's partial sum (the caller all-reduces it: ``copy_to_tp_region``).
def _local_stats(hidden, weight, labels_local, temperature):
    """(lse_r, mean_r, label_logit_r) of this rank's vocabulary shard; label_logit_r = 0 where the label is elsewhere."""
    T = hidden.shape[0]
    V = weight.shape[0]
    inside = (labels_local >= 0) & (labels_local < V)
    if hidden.is_cuda:
        dev = hidden.device
        splits = _lib.fn("vb_lmhead_num_splits")(T, V)
        scratch = torch.empty(T * splits * 4, dtype=torch.float32, device=dev)
        logp, ent, lse, mean = (torch.empty(T, dtype=torch.float32, device=dev) for _ in range(4))
        safe = torch.where(inside, labels_local, torch.full_like(labels_local, -1)).contiguous()
        rc = _lib.fn("vb_lmhead_logprob_fwd")(hidden.data_ptr(), weight.data_ptr(), safe.data_ptr(), T, hidden.shape[1], V,
                                              1.0 / temperature, scratch.data_ptr(), logp.data_ptr(), ent.data_ptr(),
                                              lse.data_ptr(), mean.data_ptr(), _lib.status_word(dev).data_ptr(),
                                              _lib.stream())
        _lib.check(rc, "vb_lmhead_logprob_fwd")
        label_logit = torch.where(inside, logp + lse, torch.zeros_like(lse))
        return lse, mean, label_logit
    logits = (hidden.float() @ weight.float().t()) / temperature
    lse = torch.logsumexp(logits, -1)
    mean = (torch.softmax(logits, -1) * logits).sum(-1)
    ll = logits.gather(-1, labels_local.clamp(0, V - 1).unsqueeze(-1)).squeeze(-1)
    return lse, mean, torch.where(inside, ll, torch.zeros_like(ll))


class _LMHeadTPFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, temperature, vocab_offset, group):
        import torch.distributed as dist

        labels_local = (labels - vocab_offset).contiguous()
        lse_r, mean_r, ll_r = _local_stats(hidden, weight, labels_local, temperature)
        m = lse_r.clone()
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        w = torch.exp(lse_r - m)
        packed = torch.stack([w, ll_r, w * mean_r])
        dist.all_reduce(packed, group=group)
        lse = m + torch.log(packed[0])
        mean = packed[2] / packed[0]
        logp = packed[1] - lse
        ent = lse - mean
        ctx.save_for_backward(hidden, weight, labels_local, lse, mean)
        ctx.temperature = temperature
        return logp, ent

    @staticmethod
    def backward(ctx, g_logp, g_ent):
        hidden, weight, labels_local, lse, mean = ctx.saved_tensors
        T, H = hidden.shape
        V = weight.shape[0]
        dev = hidden.device
        g_logp = g_logp.float().contiguous() if g_logp is not None else torch.zeros(T, device=dev)
        g_ent_t = g_ent.float().contiguous() if g_ent is not None else None
        need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        main_grad = getattr(weight, "main_grad", None)
        if not hidden.is_cuda:
            logits = (hidden.float() @ weight.float().t()) / ctx.temperature
            p = torch.exp(logits - lse[:, None])
            onehot = torch.zeros_like(p)
            inside = (labels_local >= 0) & (labels_local < V)
            onehot[inside, labels_local[inside]] = 1.0
            dl = g_logp[:, None] * (onehot - p)
            if g_ent_t is not None:
                dl = dl - g_ent_t[:, None] * p * (logits - mean[:, None])
            dl = dl / ctx.temperature
            dh = (dl @ weight.float()).to(hidden.dtype) if need_dh else None
            dw = None
            if need_dw:
                gw = dl.t() @ hidden.float()
                if main_grad is not None:
                    main_grad.add_(gw)
                else:
                    dw = gw.to(weight.dtype)
            return dh, dw, None, None, None, None
        d_hidden = torch.zeros(T, H, dtype=torch.float32, device=dev) if need_dh else None
        d_weight = None
        if need_dw:
            d_weight = main_grad if main_grad is not None else torch.zeros(V, H, dtype=torch.float32, device=dev)
        chunk = min(_DLOGITS_CHUNK, V)
        dl = torch.empty(T, chunk, dtype=torch.bfloat16, device=dev)
        fn = _lib.fn("vb_lmhead_dlogits")
        safe = torch.where((labels_local >= 0) & (labels_local < V), labels_local, torch.full_like(labels_local, -1)).contiguous()
        for off in range(0, V, chunk):
            vc = min(chunk, V - off)
            w_chunk = weight[off : off + vc]
            rc = fn(hidden.data_ptr(), w_chunk.data_ptr(), safe.data_ptr(), T, H, vc, off, 1.0 / ctx.temperature,
                    lse.data_ptr(), mean.data_ptr(), g_logp.data_ptr(), _lib.ptr(g_ent_t), dl.data_ptr(), chunk,
                    _lib.status_word(dev).data_ptr(), _lib.stream())
            _lib.check(rc, "vb_lmhead_dlogits")
            dl_v = dl[:, :vc]
            if need_dh:
                gemm(dl_v, w_chunk, b_mn=True, out=d_hidden, accumulate=True)
            if need_dw:
                gemm(dl_v, hidden, a_mn=True, b_mn=True, out=d_weight[off : off + vc], accumulate=True)
        dh = d_hidden.to(hidden.dtype) if need_dh else None
        dw = d_weight.to(weight.dtype) if (need_dw and main_grad is None) else None
        return dh, dw, None, None, None, None


def lmhead_logprob_entropy_tp(hidden: torch.Tensor, weight_shard: torch.Tensor, labels: torch.Tensor, temperature: float,
                              vocab_offset: int, group) -> tuple[torch.Tensor, torch.Tensor]:
    """Vocabulary-parallel fused lm_head: ``weight_shard [V / tp, H]`` holds the rows ``[vocab_offset, vocab_offset +
    V / tp)``; ``hidden`` and ``labels`` are replicated over ``group``. Returns the same (logprob, entropy) on every
    rank. The gradient with respect to ``hidden`` is this rank's partial sum."""
    return _LMHeadTPFn.apply(hidden.contiguous(), weight_shard, labels.contiguous().long(), float(temperature),
                             int(vocab_offset), group)


# ---------------------------------------------------------------------------------------------------------------
# The reference's call shapes over the same fused op.
def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0,
                         reduction: str = "none", dist_process_group=None) -> tuple[torch.Tensor, torch.Tensor]:
    """``(log_probs, entropy)`` of ``labels`` under ``softmax(hidden @ weight.T / temperature)`` with the argument list of
    verl/utils/kernel/linear_cross_entropy.py:38-139. ``hidden`` may be ``[B, T, H]`` with ``labels [B, T]``; with a
    ``dist_process_group`` ``weight`` is this rank's slice of the vocabulary (slices in rank order)."""
    shape = labels.shape
    h2, l1 = hidden.reshape(-1, hidden.shape[-1]), labels.reshape(-1)
    if dist_process_group is not None and torch.distributed.get_world_size(dist_process_group) > 1:
        off = torch.distributed.get_rank(dist_process_group) * weight.shape[0]
        lp, ent = lmhead_logprob_entropy_tp(h2, weight, l1, temperature, off, dist_process_group)
    else:
        lp, ent = lmhead_logprob_entropy(h2, weight, l1, temperature)
    if reduction == "mean":
        return lp.mean(), ent.mean()
    if reduction == "sum":
        return lp.sum(), ent.sum()
    return lp.view(shape), ent.view(shape)


class FusedLinearForPPO(torch.nn.Module):
    """Module form with the call shape of verl/utils/experimental/torch_functional.py:190-216. ``chunk_size`` is accepted
    and unused: the kernel tiles the vocabulary itself and never holds a ``[T, V]`` tensor."""

    def __init__(self, chunk_size: int = 512):
        super().__init__()
        self.chunk_size = chunk_size

    def forward(self, hidden_states: torch.Tensor, vocab_weights: torch.Tensor, input_ids: torch.Tensor,
                temperature: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
        return linear_cross_entropy(hidden_states, vocab_weights, input_ids.to(torch.int64), temperature)
