"""Batch assembly after generation: left-padded prompts + right-padded responses, masks and positions.

Layout contract of the reference's agent-loop post-processing (verl/experimental/agent_loop/
agent_loop.py:521-640,732-806): ``prompts [B,P]`` left-padded, ``responses [B,R]`` right-padded,
``input_ids = [prompts | responses]``, ``attention_mask``, ``position_ids`` (cumulative over the mask),
``response_mask`` (1 = model-generated token), optional ``rollout_log_probs``.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..protocol import DataProto


def assemble_rollout_batch(prompt_ids: torch.Tensor, prompt_mask: torch.Tensor, outputs: Sequence, response_length: int,
                           pad_token_id: int = 0, with_logprobs: bool = True,
                           response_masks: Optional[Sequence[Sequence[int]]] = None) -> DataProto:
    """``prompt_ids`` / ``prompt_mask``: [B,P] left-padded. ``outputs``: objects with ``token_ids`` (and
    ``log_probs``). ``response_masks`` marks model tokens (1) vs tool / user tokens (0) for multi-turn."""
    B, P = prompt_ids.shape
    R = response_length
    resp = torch.full((B, R), pad_token_id, dtype=prompt_ids.dtype)
    rmask = torch.zeros(B, R, dtype=prompt_mask.dtype)
    amask_r = torch.zeros(B, R, dtype=prompt_mask.dtype)
    lps = torch.zeros(B, R, dtype=torch.float32)
    for i, o in enumerate(outputs):
        toks = list(o.token_ids)[:R]
        n = len(toks)
        if n:
            resp[i, :n] = torch.tensor(toks, dtype=prompt_ids.dtype)
            amask_r[i, :n] = 1
            if response_masks is not None:
                rmask[i, :n] = torch.tensor(list(response_masks[i])[:n], dtype=prompt_mask.dtype)
            else:
                rmask[i, :n] = 1
            if with_logprobs and getattr(o, "log_probs", None) is not None:
                lp = list(o.log_probs)[:n]
                lps[i, : len(lp)] = torch.tensor(lp, dtype=torch.float32)
    input_ids = torch.cat([prompt_ids, resp], dim=1)
    attention_mask = torch.cat([prompt_mask, amask_r], dim=1)
    position_ids = (torch.cumsum(attention_mask, dim=1) - 1).clamp(min=0)
    tensors = {"prompts": prompt_ids, "responses": resp, "input_ids": input_ids, "attention_mask": attention_mask,
               "position_ids": position_ids, "response_mask": rmask}
    if with_logprobs:
        tensors["rollout_log_probs"] = lps
    return DataProto.from_dict(tensors=tensors)
