"""Tensor helpers used across trainers and workers (masked statistics, log-prob / entropy from
logits, response masks, padding helpers, LR schedules, cross-rank statistics).

Counterpart of verl/utils/torch_functional.py; the materialised-logits functions here are the
oracle and CPU path, the GPU hot path is the fused lm_head kernel in :mod:`verl_b200.ops`.
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch.optim.lr_scheduler import LambdaLR


# ----------------------------------------------------------------- masked statistics
def masked_sum(values: torch.Tensor, mask: torch.Tensor, axis=None) -> torch.Tensor:
    v = torch.where(mask.bool(), values, torch.zeros_like(values))  # NaNs outside the mask do not leak
    return v.sum(axis) if axis is not None else v.sum()


def masked_mean(values: torch.Tensor, mask: torch.Tensor, axis=None) -> torch.Tensor:
    s = masked_sum(values, mask, axis)
    return s / (mask.sum(axis) + 1e-8) if axis is not None else s / (mask.sum() + 1e-8)


def masked_var(values: torch.Tensor, mask: torch.Tensor, unbiased: bool = True) -> torch.Tensor:
    mean = masked_mean(values, mask)
    var = masked_mean((values - mean) ** 2, mask)
    if unbiased:
        n = mask.sum()
        if n == 0:
            raise ValueError("At least one element in the mask has to be 1.")
        if n == 1:
            raise ValueError("The sum of the mask is one, which can cause a division by zero.")
        var = var * (n / (n - 1))
    return var


def masked_whiten(values: torch.Tensor, mask: torch.Tensor, shift_mean: bool = True) -> torch.Tensor:
    mean, var = masked_mean(values, mask), masked_var(values, mask)
    out = (values - mean) * torch.rsqrt(var + 1e-8)
    if not shift_mean:
        out = out + mean
    return out


def clip_by_value(x, tensor_min, tensor_max):
    return torch.max(torch.min(x, tensor_max), tensor_min)


# -------------------------------------------------------------- logits -> statistics
def logprobs_from_logits(logits: torch.Tensor, labels: torch.Tensor, inplace_backward: bool = True) -> torch.Tensor:
    """log_softmax(logits)[labels] without keeping a full fp32 log-softmax when not needed."""
    if logits.dtype in (torch.float32, torch.float64):
        picked = torch.gather(logits, -1, labels.unsqueeze(-1)).squeeze(-1)
        return picked - torch.logsumexp(logits, dim=-1)
    out = []
    flat = logits.reshape(-1, logits.shape[-1])
    lab = labels.reshape(-1)
    for row, l in zip(flat.split(4096), lab.split(4096)):  # row-chunked for half precision
        lsm = F.log_softmax(row.float(), dim=-1)
        out.append(lsm.gather(-1, l.unsqueeze(-1)).squeeze(-1))
    return torch.cat(out).reshape(labels.shape)


def logprobs_from_logits_v2(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    return logprobs_from_logits(logits, labels)


def entropy_from_logits(logits: torch.Tensor) -> torch.Tensor:
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    return lse - (torch.softmax(lf, dim=-1) * lf).sum(-1)


def entropy_from_logits_with_chunking(logits: torch.Tensor, chunk_size: int = 2048) -> torch.Tensor:
    flat = logits.reshape(-1, logits.shape[-1])
    out = torch.cat([entropy_from_logits(c) for c in flat.split(chunk_size)])
    return out.reshape(logits.shape[:-1])


def calculate_sum_pi_squared_from_logits(logits: torch.Tensor) -> torch.Tensor:
    """sum_v softmax(logits)_v^2 per position (optimal-token-baseline estimators)."""
    p = torch.softmax(logits.float(), dim=-1)
    return (p * p).sum(-1)


# ------------------------------------------------------------------- masks / padding
def get_response_mask(response_id: torch.Tensor, eos_token: int | list[int] = 2, dtype=torch.int64) -> torch.Tensor:
    """1 up to and including the first EOS, 0 after (e.g. [a,b,eos,c] -> [1,1,1,0])."""
    eos = torch.as_tensor(eos_token if isinstance(eos_token, (list, tuple)) else [eos_token], device=response_id.device)
    is_eos = torch.isin(response_id, eos)
    after = (torch.cumsum(is_eos, dim=1) - is_eos.long()) > 0
    return (~after).to(dtype)


def get_eos_mask(response_id, eos_token=2, dtype=torch.int64):
    return get_response_mask(response_id, eos_token, dtype)


def pad_sequence_to_length(t: torch.Tensor, max_len: int, pad_value, left_pad: bool = False) -> torch.Tensor:
    if t.shape[-1] >= max_len:
        return t
    pad = (max_len - t.shape[-1], 0) if left_pad else (0, max_len - t.shape[-1])
    return F.pad(t, pad, "constant", pad_value)


def pad_2d_list_to_length(rows: list[list[int]], pad_token_id: int, max_length: Optional[int] = None) -> torch.Tensor:
    n = max(len(r) for r in rows) if rows else 0
    target = max(n, max_length) if max_length is not None else n
    return torch.tensor([list(r) + [pad_token_id] * (target - len(r)) for r in rows])


def compute_position_id_with_mask(mask: torch.Tensor) -> torch.Tensor:
    return torch.clip(torch.cumsum(mask, dim=-1) - 1, min=0, max=None)


def postprocess_data(input_ids, attention_mask, max_length: int, pad_token_id: int, left_pad=True, truncation="error"):
    """Pad or truncate tokenised prompts to ``max_length`` (truncation in {left,right,middle,error})."""
    assert truncation in ("left", "right", "middle", "error")
    L = input_ids.shape[-1]
    if L < max_length:
        input_ids = pad_sequence_to_length(input_ids, max_length, pad_token_id, left_pad)
        attention_mask = pad_sequence_to_length(attention_mask, max_length, 0, left_pad)
    elif L > max_length:
        if truncation == "left":
            input_ids, attention_mask = input_ids[:, -max_length:], attention_mask[:, -max_length:]
        elif truncation == "right":
            input_ids, attention_mask = input_ids[:, :max_length], attention_mask[:, :max_length]
        elif truncation == "middle":
            lh = max_length // 2
            rh = max_length - lh
            input_ids = torch.cat([input_ids[:, :lh], input_ids[:, -rh:]], dim=-1)
            attention_mask = torch.cat([attention_mask[:, :lh], attention_mask[:, -rh:]], dim=-1)
        else:
            raise NotImplementedError(f"sequence_length={L} is larger than max_length={max_length}")
    return input_ids, attention_mask


def tokenize_and_postprocess_data(prompt: str, tokenizer, max_length: int, pad_token_id: int, left_pad=True,
                                  truncation="error"):
    enc = tokenizer(prompt, return_tensors="pt", add_special_tokens=False)
    return postprocess_data(enc["input_ids"], enc["attention_mask"], max_length, pad_token_id, left_pad, truncation)


def remove_pad_token(input_ids: torch.Tensor, attention_mask: torch.Tensor) -> list[list[int]]:
    return [ids[len(ids) - int(m.sum()):].tolist() for ids, m in zip(input_ids, attention_mask)]


# ------------------------------------------------------------------------ schedules
def get_constant_schedule_with_warmup(optimizer, num_warmup_steps: int, last_epoch: int = -1):
    def fn(step):
        return min(1.0, float(step) / float(max(1, num_warmup_steps)))

    return LambdaLR(optimizer, fn, last_epoch)


def get_cosine_schedule_with_warmup(optimizer, num_warmup_steps: int, num_training_steps: int,
                                    min_lr_ratio: float = 0.0, num_cycles: float = 0.5, last_epoch: int = -1,
                                    init_lr_ratio: Optional[float] = None):
    min_lr_ratio = 0.0 if min_lr_ratio is None else min_lr_ratio
    init_lr_ratio = 0.0 if init_lr_ratio is None else init_lr_ratio
    coef, intercept = (1 - min_lr_ratio) * 0.5, (1 + min_lr_ratio) * 0.5

    def fn(step):
        if step < num_warmup_steps:
            return init_lr_ratio + (1.0 - init_lr_ratio) * (float(step) / float(max(1, num_warmup_steps)))
        prog = float(step - num_warmup_steps) / float(max(1, num_training_steps - num_warmup_steps))
        return max(min_lr_ratio, math.cos(math.pi * float(num_cycles) * 2.0 * prog) * coef + intercept)

    return LambdaLR(optimizer, fn, last_epoch)


def get_wsd_schedule_with_warmup(optimizer, num_warmup_steps: int, num_training_steps: int, min_lr_ratio: float = 0.0,
                                 stable_ratio: float = 0.9, last_epoch: int = -1):
    """Warmup -> stable -> cosine decay."""
    remain = num_training_steps - num_warmup_steps
    n_stable = int(remain * stable_ratio)
    n_decay = max(1, remain - n_stable)

    def fn(step):
        if step < num_warmup_steps:
            return float(step) / float(max(1, num_warmup_steps))
        if step < num_warmup_steps + n_stable:
            return 1.0
        prog = min(1.0, float(step - num_warmup_steps - n_stable) / float(n_decay))
        return max(min_lr_ratio, min_lr_ratio + (1 - min_lr_ratio) * 0.5 * (1.0 + math.cos(math.pi * prog)))

    return LambdaLR(optimizer, fn, last_epoch)


# ------------------------------------------------------------------- cross-rank stats
def distributed_mean_max_min_std(local: torch.Tensor, compute_max=True, compute_min=True, compute_std=True):
    """Global mean / max / min / std of a 1-D tensor spread over the default process group."""
    n = torch.tensor([local.numel()], dtype=torch.float64, device=local.device)
    s = local.double().sum().reshape(1)
    dist.all_reduce(n)
    dist.all_reduce(s)
    mean = (s / n).to(local.dtype)
    mx = mn = std = None
    if compute_max:
        mx = local.max().reshape(1).clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    if compute_min:
        mn = local.min().reshape(1).clone()
        dist.all_reduce(mn, op=dist.ReduceOp.MIN)
    if compute_std:
        sq = ((local.double() - s / n) ** 2).sum().reshape(1)
        dist.all_reduce(sq)
        std = torch.sqrt(sq / (n - 1)).to(local.dtype)
    return mean.squeeze(), (mx.squeeze() if mx is not None else None), (mn.squeeze() if mn is not None else None), (
        std.squeeze() if std is not None else None)


def distributed_masked_mean(local: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    s = masked_sum(local, mask).reshape(1).double()
    n = mask.sum().reshape(1).double()
    dist.all_reduce(s)
    dist.all_reduce(n)
    return (s / n).to(local.dtype).squeeze()


# ----------------------------------------------------- log-probs from materialised logits (padded / packed layouts)
def gather_from_labels(data: torch.Tensor, label: torch.Tensor) -> torch.Tensor:
    """``data[..., label]``: the entry of the last dimension that ``label`` names, per position."""
    return torch.gather(data, -1, label.unsqueeze(-1)).squeeze(-1)


def logprobs_from_logits_naive(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    return gather_from_labels(torch.log_softmax(logits, dim=-1), labels)


def post_process_logits(input_ids, logits: torch.Tensor, temperature: float, top_k=None, top_p=None) -> torch.Tensor:
    """Temperature scaling in place (top-k / top-p warping changes the policy's support and is left to the sampler)."""
    return logits.div_(temperature) if temperature != 1.0 else logits


def log_probs_from_logits_response(input_ids: torch.Tensor, logits: torch.Tensor, response_length: int) -> torch.Tensor:
    """``logits = model(input_ids)`` ``[B, S, V]`` -> log-probs of the last ``response_length`` tokens ``[B, R]``
    (position t predicts token t + 1)."""
    return logprobs_from_logits(logits[:, -response_length - 1 : -1], input_ids[:, -response_length:])


def get_unpad_data(attention_mask: torch.Tensor):
    """(flat indices of the kept tokens, cu_seqlens int32 [B + 1], longest sequence) of a padded batch."""
    lens = attention_mask.sum(dim=-1, dtype=torch.int32)
    idx = torch.nonzero(attention_mask.flatten(), as_tuple=False).flatten()
    cu = torch.nn.functional.pad(torch.cumsum(lens, 0, dtype=torch.int32), (1, 0))
    return idx, cu, int(lens.max().item())


def log_probs_from_logits_all_rmpad(input_ids_rmpad: torch.Tensor, logits_rmpad: torch.Tensor, indices: torch.Tensor,
                                    batch_size: int, seqlen: int, response_length: int) -> torch.Tensor:
    """Packed ids ``[1, nnz]`` (or ``[nnz]``) and packed logits ``[nnz, V]`` with the flat ``indices`` of the packed
    tokens in the ``[B, S]`` layout -> response log-probs ``[B, R]`` (zeros at padding). Within the packed stream token
    t + 1 is the label of position t; the roll's wrap-around at a sequence's last token lands on a position that is
    never a response row of the padded layout."""
    ids = input_ids_rmpad.reshape(-1)
    lp = logprobs_from_logits(logits_rmpad, torch.roll(ids, -1, 0))
    full = torch.zeros(batch_size * seqlen, dtype=lp.dtype, device=lp.device)
    full[indices] = lp
    return full.view(batch_size, seqlen)[:, -response_length - 1 : -1]


def log_probs_from_logits_response_rmpad(input_ids: torch.Tensor, attention_mask: torch.Tensor, logits_rmpad: torch.Tensor,
                                         response_length: int) -> torch.Tensor:
    """Padded ids / mask ``[B, S]`` and packed logits ``[nnz, V]`` -> response log-probs ``[B, R]``."""
    b, s = input_ids.shape
    idx, _, _ = get_unpad_data(attention_mask)
    return log_probs_from_logits_all_rmpad(input_ids.reshape(-1)[idx], logits_rmpad, idx, b, s, response_length)


def compute_grad_norm(model) -> float:
    """SUM OF SQUARES of all gradients of ``model`` (take the square root for the L2 norm)."""
    return float(sum(torch.sum(torch.square(p.grad.detach().float())) for p in model.parameters() if p.grad is not None))


def broadcast_dict_tensor(tensors, src: int, group) -> None:
    import torch.distributed as dist

    for key in sorted(tensors.keys()):
        dist.broadcast(tensors[key], src=src, group=group)


def split_dict_tensor_into_batches(tensors, batch_size: int) -> list:
    n = tensors.batch_size[0]
    assert n % batch_size == 0, f"input data batch size: {n}, split batch size: {batch_size}"
    return tensors.split(batch_size)


def expand_as_nested(tensor: torch.Tensor, nested_tensor: torch.Tensor) -> torch.Tensor:
    """``tensor [B]`` -> a jagged tensor shaped like ``nested_tensor [B, j]`` whose row i repeats ``tensor[i]``."""
    assert nested_tensor.is_nested, "nested_tensor must be nested"
    assert tensor.shape[0] == nested_tensor.shape[0], f"The batch shape must be the same. Got {tensor.shape[0]} vs {nested_tensor.shape[0]}"
    offsets = nested_tensor.offsets()
    return torch.nested.nested_tensor_from_jagged(torch.repeat_interleave(tensor, offsets.diff()), offsets=offsets)


def prepare_decoder_attention_mask(attention_mask: Optional[torch.Tensor], input_shape, inputs_embeds: torch.Tensor) -> torch.Tensor:
    """Additive ``[B, 1, T, T]`` mask of a decoder: causal, and the most negative value at padded keys."""
    b, t = input_shape
    neg = torch.finfo(inputs_embeds.dtype).min
    mask = torch.zeros(b, 1, t, t, dtype=inputs_embeds.dtype, device=inputs_embeds.device)
    if t > 1:
        mask = mask.masked_fill(torch.triu(torch.ones(t, t, dtype=torch.bool, device=mask.device), 1), neg)
    if attention_mask is not None:
        mask = mask.masked_fill(~attention_mask.bool()[:, None, None, :].to(mask.device), neg)
    return mask
