"""Log-probabilities and entropy of logits whose VOCABULARY dimension is sharded over a tensor-parallel group (role of
verl/utils/megatron/tensor_parallel.py:113-188). Each rank holds ``logits[..., v0:v1]``; three small all-reduces (max,
sum-exp, the picked logit) replace gathering the vocabulary. The fused LM-head kernel path
(``verl_b200.ops.lmhead.lmhead_logprob_entropy_tp``) never materialises logits at all; these functions serve callers
that already hold sharded logits (a custom head, a reward head, tests)."""

from __future__ import annotations

import torch
import torch.distributed as dist


def _world(group) -> tuple[int, int]:
    if not (dist.is_available() and dist.is_initialized()):
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


def _allreduce(t, op, group):
    if _world(group)[1] > 1:
        dist.all_reduce(t, op=op, group=group)
    return t


class _VocabParallelLogProb(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits: torch.Tensor, labels: torch.Tensor, group):
        rank, _ = _world(group)
        v = logits.shape[-1]
        x = logits.float()
        m = _allreduce(x.amax(dim=-1), dist.ReduceOp.MAX, group)
        e = torch.exp(x - m.unsqueeze(-1))
        s = _allreduce(e.sum(dim=-1), dist.ReduceOp.SUM, group)
        local = labels - rank * v
        mine = (local >= 0) & (local < v)
        idx = local.clamp(0, v - 1).unsqueeze(-1)
        picked = _allreduce(torch.where(mine, x.gather(-1, idx).squeeze(-1), torch.zeros_like(m)), dist.ReduceOp.SUM, group)
        ctx.save_for_backward(e / s.unsqueeze(-1), idx, mine)
        ctx.in_dtype = logits.dtype
        return picked - m - torch.log(s)

    @staticmethod
    def backward(ctx, g):
        p, idx, mine = ctx.saved_tensors
        grad = -p * g.unsqueeze(-1)
        grad.scatter_add_(-1, idx, (g * mine).unsqueeze(-1))
        return grad.to(ctx.in_dtype), None, None


class _VocabParallelEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits: torch.Tensor, group):
        x = logits.float()
        m = _allreduce(x.amax(dim=-1), dist.ReduceOp.MAX, group)
        xs = x - m.unsqueeze(-1)
        e = torch.exp(xs)
        s = _allreduce(e.sum(dim=-1), dist.ReduceOp.SUM, group)
        p = e / s.unsqueeze(-1)
        mean = _allreduce((p * xs).sum(dim=-1), dist.ReduceOp.SUM, group)  # E_p[x - m]
        ent = torch.log(s) - mean
        ctx.save_for_backward(p, xs, mean)
        ctx.in_dtype = logits.dtype
        return ent

    @staticmethod
    def backward(ctx, g):
        p, xs, mean = ctx.saved_tensors
        # dH/dx_j = -p_j * ((x_j - m) - E_p[x - m])
        return (-(p * (xs - mean.unsqueeze(-1))) * g.unsqueeze(-1)).to(ctx.in_dtype), None


def vocab_parallel_log_probs_from_logits(logits: torch.Tensor, labels: torch.Tensor, group=None) -> torch.Tensor:
    """``logits [..., V / tp]`` (this rank's slice of the vocabulary, slices in rank order), ``labels [...]`` global ids
    -> ``log softmax(logits)[labels]`` in fp32, identical on every rank of ``group``."""
    return _VocabParallelLogProb.apply(logits, labels, group)


def vocab_parallel_entropy(logits: torch.Tensor, group=None) -> torch.Tensor:
    """Entropy of the softmax over the full (sharded) vocabulary, fp32, identical on every rank of ``group``."""
    return _VocabParallelEntropy.apply(logits, group)


def vocab_parallel_log_probs_from_logits_response_rmpad(input_ids: torch.Tensor, attention_mask: torch.Tensor,
                                                        logits_rmpad: torch.Tensor, response_length: int, group=None):
    """Packed (padding removed) sharded logits ``[total_nnz, V / tp]`` of a ``[B, S]`` batch -> log-probs of the response
    tokens ``[B, response_length]`` (zeros at padded positions). The label of position t is token t + 1."""
    b, s = input_ids.shape
    keep = attention_mask.bool().reshape(-1)
    nxt = torch.roll(input_ids, shifts=-1, dims=1).reshape(-1)[keep]
    lp = vocab_parallel_log_probs_from_logits(logits_rmpad, nxt, group)
    full = torch.zeros(b * s, dtype=lp.dtype, device=lp.device)
    full[keep] = lp
    return full.view(b, s)[:, -response_length - 1:-1]


def is_tensor_parallel_param(param) -> bool:
    return bool(getattr(param, "tensor_model_parallel", False))


def get_tensor_parallel_partition_dim(param) -> int:
    assert is_tensor_parallel_param(param)
    return int(param.partition_dim)


def get_tensor_parallel_partition_stride(param) -> int:
    assert is_tensor_parallel_param(param)
    return int(getattr(param, "partition_stride", 1))


def pad_to_sequence_parallel(unpad_tokens: torch.Tensor, sp_world_size: int) -> torch.Tensor:
    """Pads dim 0 of a packed token tensor with zeros up to a multiple of the sequence-parallel size."""
    pad = (-unpad_tokens.shape[0]) % max(sp_world_size, 1)
    if pad == 0:
        return unpad_tokens
    return torch.cat([unpad_tokens, unpad_tokens.new_zeros((pad,) + tuple(unpad_tokens.shape[1:]))], dim=0)
