"""Shared-prefix packing of the n samples of one prompt (role of verl/trainer/ppo/prefix_grouper_utils.py:1-235).

GRPO evaluates n responses per prompt; in the padded layout each of them repeats the prompt tokens in the log-prob
and update passes. ``build_prefix_groups`` finds the runs of samples that share a prompt (same ``uid`` or the same
prompt tokens) and ``pack_with_shared_prefix`` lays a group out as ONE packed sequence
``[prompt, response_0, response_1, ...]`` together with a position-id vector (every response continues after the
prompt) and a segment table for a prefix-sharing attention mask: response i attends to the prompt and to itself.
``unpack_shared_prefix`` scatters per-token results of the packed stream back to ``[B, R]``.

The native varlen attention kernel does not take a prefix-sharing mask; the engine falls back to repeating the
prompt unless ``use_prefix_grouper`` finds an attention backend for it, so these helpers are currently the data
layout half of the feature (and are exact for models evaluated with :func:`prefix_shared_attention_reference`).
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch


@dataclass
class PrefixGroup:
    rows: list[int]          # sample indices of the batch that share the prompt
    prompt: torch.Tensor     # [P] prompt tokens without padding
    responses: list[torch.Tensor]


def build_prefix_groups(prompts: torch.Tensor, responses: torch.Tensor, attention_mask: torch.Tensor, uid=None) -> list[PrefixGroup]:
    """``prompts`` [B, P] left padded, ``responses`` [B, R] right padded, ``attention_mask`` [B, P + R]."""
    B, P = prompts.shape
    keys = []
    for i in range(B):
        if uid is not None:
            keys.append(str(uid[i]))
        else:
            keys.append(prompts[i][attention_mask[i, :P].bool()].numpy().tobytes())
    groups: dict = {}
    for i, k in enumerate(keys):
        groups.setdefault(k, []).append(i)
    out = []
    for rows in groups.values():
        i0 = rows[0]
        prompt = prompts[i0][attention_mask[i0, :P].bool()]
        resp = [responses[i][attention_mask[i, P:].bool()] for i in rows]
        out.append(PrefixGroup(rows, prompt, resp))
    return out


def pack_with_shared_prefix(groups: list[PrefixGroup]):
    """Returns (input_ids [T], position_ids [T], cu_seqlens [G+1], segments [T] with 0 = prompt and i+1 = response i,
    index [(row, j)] -> packed position of response token j of sample row)."""
    ids, pos, seg, cu, where = [], [], [], [0], {}
    for g in groups:
        p = g.prompt
        base = cu[-1]
        ids.append(p)
        pos.append(torch.arange(p.numel()))
        seg.append(torch.zeros(p.numel(), dtype=torch.long))
        off = p.numel()
        for i, (row, r) in enumerate(zip(g.rows, g.responses)):
            ids.append(r)
            pos.append(torch.arange(p.numel(), p.numel() + r.numel()))
            seg.append(torch.full((r.numel(),), i + 1, dtype=torch.long))
            where[row] = (base + off, r.numel())
            off += r.numel()
        cu.append(base + off)
    return torch.cat(ids), torch.cat(pos), torch.tensor(cu, dtype=torch.int32), torch.cat(seg), where


def prefix_sharing_mask(segments: torch.Tensor, cu_seqlens: torch.Tensor) -> torch.Tensor:
    """Boolean [T, T] mask: causal, same packed group, and key in the prompt or in the query's own response."""
    T = segments.numel()
    grp = torch.zeros(T, dtype=torch.long)
    b = cu_seqlens.tolist()
    for gi, (s, e) in enumerate(zip(b[:-1], b[1:])):
        grp[s:e] = gi
    i = torch.arange(T)
    causal = i[None, :] <= i[:, None]
    same = grp[None, :] == grp[:, None]
    ok = (segments[None, :] == 0) | (segments[None, :] == segments[:, None])
    return causal & same & ok


def unpack_shared_prefix(values: torch.Tensor, where: dict, batch_size: int, response_length: int, shift: int = 1) -> torch.Tensor:
    """Per-token values of the packed stream -> [B, R]. With ``shift = 1`` the value for response token j is read at
    the position that predicts it (one to the left; the first response token is predicted by the last prompt token,
    which the caller reads separately through ``first_token_positions``)."""
    out = torch.zeros(batch_size, response_length, dtype=values.dtype)
    for row, (start, n) in where.items():
        if n > shift:
            out[row, shift:n] = values[start : start + n - shift]
    return out


def prefix_saving(groups: list[PrefixGroup]) -> float:
    """Fraction of tokens saved against repeating the prompt for every sample."""
    repeated = sum(len(g.rows) * g.prompt.numel() + sum(r.numel() for r in g.responses) for g in groups)
    packed = sum(g.prompt.numel() + sum(r.numel() for r in g.responses) for g in groups)
    return 1.0 - packed / max(repeated, 1)
