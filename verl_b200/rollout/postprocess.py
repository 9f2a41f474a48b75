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
    first = next((o for o in outputs if getattr(o, "routed_experts", None) is not None), None)
    if first is not None:
        # mixture-of-experts rollouts that record their routing: [B, P + R, layers, top-k] aligned with input_ids (zeros
        # where a token was never an input of the model: padding, and the last token of a response)
        import numpy as np

        routed = torch.zeros((B, P + R) + tuple(first.routed_experts.shape[1:]), dtype=torch.int16)
        for i, o in enumerate(outputs):
            rec = getattr(o, "routed_experts", None)
            if rec is None:
                continue
            rec = torch.from_numpy(np.ascontiguousarray(rec))
            n_p = int(prompt_mask[i].sum())
            n_r = min(rec.shape[0] - n_p, R)
            routed[i, P - n_p : P] = rec[:n_p]
            if n_r > 0:
                routed[i, P : P + n_r] = rec[n_p : n_p + n_r]
        tensors["routed_experts"] = routed
    return DataProto.from_dict(tensors=tensors)
