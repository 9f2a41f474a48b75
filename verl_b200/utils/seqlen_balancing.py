"""Sequence-length balancing: split a batch into k parts of near-equal workload.

Counterpart of verl/utils/seqlen_balancing.py (``karmarkar_karp`` :49, ``greedy_partition`` :175,
``get_seqlen_balanced_partitions`` :213, ``rearrange_micro_batches`` :348, ``prepare_dynamic_batch``
:443, ``restore_dynamic_batch`` :482). The workload of a sequence of length s is
``24576 * s + s^2`` (linear layers + attention, :27). The partitioner here is the largest-
differencing method written over a heap of k-tuples.
"""

from __future__ import annotations

import heapq
from typing import Optional

import torch
import torch.distributed as dist

from ..protocol import DataProto


def calculate_workload(seqlen_list: torch.Tensor) -> torch.Tensor:
    return 24576 * seqlen_list + seqlen_list ** 2


def karmarkar_karp(seqlen_list: list[int], k_partitions: int, equal_size: bool) -> list[list[int]]:
    """Largest differencing method. Each state is k bins (sum, items) sorted by sum; the two states with
    the largest spread are merged by pairing the heaviest bins of one with the lightest of the other."""
    n = len(seqlen_list)
    order = sorted(range(n), key=lambda i: seqlen_list[i])
    states = []  # heap entries: (-spread, tiebreak, bins) with bins sorted descending by sum
    tick = 0

    def push(bins):
        nonlocal tick
        bins.sort(key=lambda b: -b[0])
        heapq.heappush(states, (-(bins[0][0] - bins[-1][0]), tick, bins))
        tick += 1

    if equal_size:
        assert n % k_partitions == 0, f"{n} % {k_partitions} != 0"
        for off in range(0, n, k_partitions):
            push([(seqlen_list[i], [i]) for i in order[off : off + k_partitions]])
    else:
        for i in order:
            push([(seqlen_list[i], [i])] + [(0, []) for _ in range(k_partitions - 1)])
    while len(states) > 1:
        _, _, a = heapq.heappop(states)
        _, _, b = heapq.heappop(states)
        merged = [(a[j][0] + b[k_partitions - 1 - j][0], a[j][1] + b[k_partitions - 1 - j][1])
                  for j in range(k_partitions)]
        push(merged)
    bins = states[0][2]
    parts = [sorted(items) for _, items in bins]
    if equal_size:
        for p in parts:
            assert len(p) * k_partitions == n, f"{len(p)} * {k_partitions} != {n}"
    return parts


def greedy_partition(seqlen_list: list[int], k_partitions: int, equal_size: bool) -> list[list[int]]:
    bias = sum(seqlen_list) + 1 if equal_size else 0
    parts = [[] for _ in range(k_partitions)]
    sums = [0] * k_partitions
    for i in sorted(range(len(seqlen_list)), key=lambda i: -seqlen_list[i]):
        j = min(range(k_partitions), key=lambda j: sums[j])
        parts[j].append(i)
        sums[j] += seqlen_list[i] + bias
    if equal_size:
        for p in parts:
            assert len(p) * k_partitions == len(seqlen_list)
    return parts


def get_seqlen_balanced_partitions(seqlen_list: list[int], k_partitions: int, equal_size: bool) -> list[list[int]]:
    """Indices of ``seqlen_list`` split into ``k_partitions`` lists with balanced sums; every index appears once."""
    assert len(seqlen_list) >= k_partitions, f"number of items:[{len(seqlen_list)}] < k_partitions:[{k_partitions}]"
    parts = karmarkar_karp(seqlen_list, k_partitions, equal_size)
    assert len(parts) == k_partitions
    seen = set()
    out = []
    for p in parts:
        assert len(p) > 0, "empty partition"
        seen.update(p)
        out.append(sorted(p))
    assert seen == set(range(len(seqlen_list)))
    return out


def get_group_balanced_partitions(seqlen_list: list[int], group_ids: list, k_partitions: int) -> list[list[int]]:
    """Like the above but samples sharing a group id stay in the same partition."""
    groups: dict = {}
    for i, g in enumerate(group_ids):
        groups.setdefault(g, []).append(i)
    keys = list(groups.keys())
    loads = [sum(seqlen_list[i] for i in groups[k]) for k in keys]
    parts = get_seqlen_balanced_partitions(loads, k_partitions, equal_size=False)
    return [sorted(i for gi in p for i in groups[keys[gi]]) for p in parts]


def log_seqlen_unbalance(seqlen_list: list[int], partitions: list[list[int]], prefix: str) -> dict:
    k = len(partitions)
    n = len(seqlen_list)
    per = n // k
    naive = [sum(seqlen_list[i * per : (i + 1) * per]) for i in range(k)]
    bal = [sum(seqlen_list[i] for i in p) for p in partitions]
    return {f"{prefix}/min": min(naive), f"{prefix}/max": max(naive), f"{prefix}/minmax_diff": max(naive) - min(naive),
            f"{prefix}/balanced_min": min(bal), f"{prefix}/balanced_max": max(bal), f"{prefix}/mean": sum(naive) / k}


def ceildiv(a, b):
    return -(a // -b)


def roundup_divisible(a, b):
    return ((a + b - 1) // b) * b


def rearrange_micro_batches(batch, max_token_len: int, dp_group=None, num_batches_divided_by=None,
                            same_micro_num_in_dp: bool = True, min_num_micro_batch: Optional[int] = None,
                            use_dynamic_bsz_balance: bool = True):
    """Split a TensorDict-like ``batch`` (needs ``attention_mask``) into micro-batches whose total
    token count is at most ``max_token_len``. Returns (micro_batches, index lists)."""
    ids = batch["input_ids"] if "input_ids" in batch.keys() else None
    if ids is not None and ids.is_nested:  # the no-padding layout: one jagged row per sample, no mask
        seq_lens = ids.offsets().diff()
        max_seq_len, mask = int(seq_lens.max()), seq_lens
    else:
        mask = batch["attention_mask"]
        max_seq_len = mask.shape[-1]
        seq_lens = mask.sum(dim=1)
    assert max_token_len >= max_seq_len, f"max_token_len must be greater than the sequence length. Got {max_token_len=} and {max_seq_len=}"
    total = int(seq_lens.sum())
    num = min(len(seq_lens), ceildiv(total, max_token_len))
    if min_num_micro_batch is not None:
        num = max(min_num_micro_batch, num)
    if dist.is_available() and dist.is_initialized() and same_micro_num_in_dp:
        t = torch.tensor([num], device=mask.device if mask.is_cuda else "cpu")
        if dist.get_backend(dp_group) == "nccl" and not t.is_cuda:
            t = t.cuda()
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=dp_group)
        num = int(t.item())
    if num_batches_divided_by is not None:
        num = roundup_divisible(num, num_batches_divided_by)
    num = min(num, len(seq_lens)) if len(seq_lens) >= 1 else num
    lens = seq_lens.tolist()
    parts = get_seqlen_balanced_partitions(lens, num, equal_size=False)
    if use_dynamic_bsz_balance:
        parts.sort(key=lambda p: (sum(calculate_workload(torch.tensor([lens[i] for i in p]))).item(), min(p)),
                   reverse=True)
    micro = [batch[torch.tensor(p)] for p in parts]
    return micro, parts


def get_reverse_idx(idx_map: list[int]) -> list[int]:
    rev = [0] * len(idx_map)
    for i, j in enumerate(idx_map):
        rev[j] = i
    return rev


def prepare_dynamic_batch(data: DataProto, max_token_len: int, dp_group=None, num_batches_divided_by=None,
                          same_micro_num_in_dp: bool = True, min_num_micro_batch=None,
                          use_dynamic_bsz_balance: bool = True):
    """DataProto -> (list of micro DataProtos, index lists); non-tensor columns follow their rows."""
    batch, idx = rearrange_micro_batches(data.batch, max_token_len, dp_group, num_batches_divided_by,
                                         same_micro_num_in_dp, min_num_micro_batch, use_dynamic_bsz_balance)
    out = []
    for i, b in enumerate(batch):
        nt = {k: v[idx[i]] for k, v in data.non_tensor_batch.items()}
        out.append(DataProto(batch=b, non_tensor_batch=nt, meta_info=data.meta_info))
    return out, idx


def restore_dynamic_batch(data: torch.Tensor, batch_idx_list: list[list[int]]) -> torch.Tensor:
    """Undo the row permutation introduced by :func:`prepare_dynamic_batch`."""
    flat = [i for p in batch_idx_list for i in p]
    assert len(flat) == data.size(0), f"{len(flat)} vs. {data.size()}"
    rev = torch.tensor(get_reverse_idx(flat), dtype=torch.long, device=data.device)
    if data.is_nested:
        rows = list(data.unbind(0))
        return torch.nested.as_nested_tensor([rows[i] for i in rev.tolist()], layout=torch.jagged)
    return data[rev]
