"""Shared-prefix packing of the n samples of one prompt (role of verl/trainer/ppo/prefix_grouper_utils.py:1-235).

GRPO evaluates n responses per prompt; in the padded layout each of them repeats the prompt tokens in the log-prob
and update passes. ``build_prefix_groups`` finds the runs of samples that share a prompt (same ``uid`` or the same
prompt tokens) and ``pack_with_shared_prefix`` lays a group out as ONE packed sequence
``[prompt, response_0, response_1, ...]`` together with a position-id vector (every response continues after the
prompt) and a segment table for a prefix-sharing attention mask: response i attends to the prompt and to itself.
``unpack_shared_prefix`` scatters per-token results of the packed stream back to ``[B, R]``.

Attention backend: :func:`shared_prefix_batch` lays a micro-batch out as ``[distinct prompts..., responses...]`` and
``models/transformer.py::Attention._attend_shared_prefix`` evaluates it with the ordinary varlen kernels (prompts
causally; every response against its prompt's keys followed by its own, through the key-stream form of the forward
kernel). That path is FORWARD ONLY (``compute_log_prob`` of the actor and of the reference policy with
``use_prefix_grouper``): the backward kernels take one boundary table for queries and keys, so ``update_policy``
keeps repeating the prompt.
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


def shared_prefix_batch(input_ids: torch.Tensor, attention_mask: torch.Tensor, response_length: int):
    """Left-padded prompts / right-padded responses ``[b, P + R]`` -> the shared-prefix packed stream.

    Returns ``(packed, rows, labels, bj, saving)`` with the meaning of ``NativeEngine.response_rows``: ``rows[i]`` is
    the packed position whose hidden state predicts response token ``bj[i] = (sample, j)`` (the LAST prompt token of
    the sample's group for j = 0), ``labels[i]`` that token. ``saving`` = fraction of tokens not evaluated. Samples with
    identical prompt tokens form a group; the positions of a response continue after its prompt."""
    from ...models.transformer import PackedBatch

    dev = input_ids.device
    b, S = input_ids.shape
    P = S - response_length
    ids_c, mask_c = input_ids.cpu(), attention_mask.cpu().bool()
    groups: dict = {}
    prompts = []
    for i in range(b):
        pt = ids_c[i, :P][mask_c[i, :P]]
        key = pt.numpy().tobytes()
        if key not in groups:
            groups[key] = len(prompts)
            prompts.append(pt)
    gid = [groups[ids_c[i, :P][mask_c[i, :P]].numpy().tobytes()] for i in range(b)]
    plen = [int(p.numel()) for p in prompts]
    p_off = [0]
    for n in plen:
        p_off.append(p_off[-1] + n)
    Tp = p_off[-1]
    resp = [ids_c[i, P:][mask_c[i, P:]] for i in range(b)]
    rlen = [int(r.numel()) for r in resp]
    r_off = [0]
    for n in rlen:
        r_off.append(r_off[-1] + n)
    ids = torch.cat(prompts + resp)
    pos = torch.cat([torch.arange(n) for n in plen] + [torch.arange(rlen[i]) + plen[gid[i]] for i in range(b)])
    k_gather = torch.cat([torch.cat([torch.arange(plen[gid[i]]) + p_off[gid[i]], torch.arange(rlen[i]) + Tp + r_off[i]])
                          for i in range(b)]) if b else torch.zeros(0, dtype=torch.long)
    klen = [plen[gid[i]] + rlen[i] for i in range(b)]
    cu = lambda lens: torch.tensor([0] + list(torch.tensor(lens, dtype=torch.long).cumsum(0).tolist()) if lens else [0], dtype=torch.int32)  # noqa: E731
    share = {"n_prompt_tokens": Tp, "cu_prompt": cu(plen).to(dev), "max_prompt": max(plen) if plen else 0,
             "cu_resp": cu(rlen).to(dev), "max_resp": max(rlen) if rlen else 0, "k_gather": k_gather.to(dev),
             "cu_k": cu(klen).to(dev), "max_k": max(klen) if klen else 0}
    packed = PackedBatch(ids.to(dev), pos.to(dev), torch.cat([cu(plen), cu(rlen)[1:] + Tp]).to(dev),
                         max(max(plen, default=0), max(rlen, default=0)), prefix_share=share)
    rows, labels, bj = [], [], []
    for i in range(b):
        for j in range(rlen[i]):
            rows.append(p_off[gid[i]] + plen[gid[i]] - 1 if j == 0 else Tp + r_off[i] + j - 1)
            bj.append((i, j))
        labels.append(resp[i])
    rows_t = torch.tensor(rows, dtype=torch.long, device=dev)
    bj_t = torch.tensor(bj, dtype=torch.long, device=dev).view(-1, 2)
    total_plain = sum(plen[gid[i]] + rlen[i] for i in range(b))
    saving = 1.0 - (Tp + r_off[-1]) / max(total_plain, 1)
    return packed, rows_t, (torch.cat(labels).to(dev) if labels else torch.zeros(0, dtype=torch.long, device=dev)), bj_t, saving
