"""Padding <-> packed layout helpers (verl/utils/attention_utils.py: the reference forwards these to flash_attn's
``bert_padding``; these are the same operations in plain torch)."""

from __future__ import annotations

import torch
from einops import rearrange  # noqa: F401  (re-exported, as the reference does)


def index_first_axis(x: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    return x.reshape(x.shape[0], -1).index_select(0, indices).reshape(-1, *x.shape[1:])


def unpad_input(hidden_states: torch.Tensor, attention_mask: torch.Tensor, unused_mask=None):
    """[B, S, ...] -> ([T, ...], indices, cu_seqlens, max_seqlen, seqlens_used)."""
    all_mask = attention_mask if unused_mask is None else attention_mask + unused_mask
    seqlens = all_mask.sum(-1, dtype=torch.int32)
    used = attention_mask.sum(-1, dtype=torch.int32)
    indices = torch.nonzero(all_mask.flatten(), as_tuple=False).flatten()
    cu = torch.nn.functional.pad(torch.cumsum(seqlens, 0, dtype=torch.int32), (1, 0))
    flat = hidden_states.reshape(-1, *hidden_states.shape[2:])
    return index_first_axis(flat, indices), indices, cu, int(seqlens.max()) if seqlens.numel() else 0, used


def pad_input(hidden_states: torch.Tensor, indices: torch.Tensor, batch: int, seqlen: int) -> torch.Tensor:
    out = hidden_states.new_zeros(batch * seqlen, *hidden_states.shape[1:])
    out[indices] = hidden_states
    return out.reshape(batch, seqlen, *hidden_states.shape[1:])
