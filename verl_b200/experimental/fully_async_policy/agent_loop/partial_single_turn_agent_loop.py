"""Single-turn agent loop whose generation can be interrupted and resumed
(verl/experimental/fully_async_policy/agent_loop/partial_single_turn_agent_loop.py:28-121).

In the fully asynchronous pipeline a weight update aborts the requests in flight. A cancelled sample comes back with
``extra_fields["is_cancel"] = True``; passing that output again (``output=...``) continues it under the new weights:
the prompt sent to the engine is prompt + partial response (a prefix-cache hit when the cache survived), and tokens
and log-probs are appended. ``param_version_start`` / ``param_version_end`` record which weights produced it."""

from __future__ import annotations

import time
from typing import Any, Optional
from uuid import uuid4

from ...agent_loop.agent_loop import AgentLoopBase, AgentLoopMetrics, AgentLoopOutput, register


@register("partial_single_turn_agent")
class PartialSingleTurnAgentLoop(AgentLoopBase):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        rc = self.config.actor_rollout_ref.rollout
        self.prompt_length, self.response_length = int(rc.prompt_length), int(rc.response_length)

    async def run(self, sampling_params: dict[str, Any], **kwargs) -> AgentLoopOutput:
        prev: Optional[AgentLoopOutput] = kwargs.get("output")
        version = int(kwargs.get("param_version", 0))
        version_start, spent = version, 0.0
        if prev is None:
            prompt_ids = await self.apply_chat_template(kwargs["raw_prompt"])
            request_prompt = prompt_ids
        elif prev.extra_fields.get("is_cancel", False):
            prompt_ids = prev.prompt_ids
            request_prompt = list(prev.prompt_ids) + list(prev.response_ids)
            version_start = prev.extra_fields.get("param_version_start", version)
            spent = prev.metrics.generate_sequences
        else:
            return prev  # finished earlier: nothing to resume
        sp = dict(sampling_params)
        done = len(prev.response_ids) if prev is not None else 0
        sp["max_tokens"] = max(0, min(int(sp.get("max_tokens", self.response_length)), self.response_length) - done)
        t0 = time.perf_counter()
        ids, lps, cancelled = await self.server_manager.generate_for_partial(
            uuid4().hex, prompt_ids=request_prompt, sampling_params=sp)
        spent += time.perf_counter() - t0
        if prev is not None:
            ids = list(prev.response_ids) + ids
            lps = list(prev.response_logprobs or []) + lps
        if len(ids) >= self.response_length:
            cancelled = False
        ids = ids[: self.response_length]
        return AgentLoopOutput(prompt_ids=prompt_ids, response_ids=ids, response_mask=[1] * len(ids),
                               response_logprobs=lps[: self.response_length] if lps else None, num_turns=2,
                               metrics=AgentLoopMetrics(generate_sequences=spent),
                               extra_fields={"is_cancel": cancelled, "param_version_start": version_start,
                                             "param_version_end": version})
