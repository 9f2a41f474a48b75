"""Segment statistics over prompt groups (samples that share a ``uid``).

Counterpart of verl/utils/groupwise.py (``as_torch_index``, ``group_mean_std``): group ids of
any hashable type are mapped to dense ``0..G-1`` indices once, after which every per-group
statistic is an ``index_add_`` / ``bincount`` on the device.
"""

from __future__ import annotations

import numpy as np
import torch


def group_index(index, device=None) -> tuple[torch.Tensor, int]:
    """Dense int64 group ids for ``index`` (np.ndarray of any dtype, list, or tensor) and the group count."""
    if isinstance(index, torch.Tensor):
        uniq, inv = torch.unique(index, return_inverse=True)
        return inv.to(device=device, dtype=torch.long), int(uniq.numel())
    arr = np.asarray(index)
    if arr.dtype == object:
        table: dict = {}
        inv_np = np.fromiter((table.setdefault(x, len(table)) for x in arr.tolist()), dtype=np.int64, count=arr.shape[0])
        n = len(table)
    else:
        uniq, inv_np = np.unique(arr, return_inverse=True)
        n = int(uniq.shape[0])
    return torch.from_numpy(np.ascontiguousarray(inv_np)).to(device=device, dtype=torch.long), n


as_torch_index = group_index


def group_mean_std(scores: torch.Tensor, inv: torch.Tensor, n_groups: int, unbiased: bool = True):
    """Per-sample (group mean, group std, group count). Groups of size 1 get mean 0 and std 1
    (the convention of the GRPO-family estimators)."""
    s = scores.to(torch.float32)
    cnt = torch.bincount(inv, minlength=n_groups).to(s.dtype)
    tot = torch.zeros(n_groups, dtype=s.dtype, device=s.device).index_add_(0, inv, s)
    mean = tot / cnt.clamp(min=1)
    dev2 = torch.zeros(n_groups, dtype=s.dtype, device=s.device).index_add_(0, inv, (s - mean[inv]) ** 2)
    denom = (cnt - 1).clamp(min=1) if unbiased else cnt.clamp(min=1)
    std = torch.sqrt(dev2 / denom)
    single = cnt <= 1
    mean = torch.where(single, torch.zeros_like(mean), mean)
    std = torch.where(single, torch.ones_like(std), std)
    return mean[inv].to(scores.dtype), std[inv].to(scores.dtype), cnt[inv]
