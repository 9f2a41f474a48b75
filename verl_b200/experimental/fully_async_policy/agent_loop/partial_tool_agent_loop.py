"""Tool-calling agent loop whose generations can be interrupted and resumed
(verl/experimental/fully_async_policy/agent_loop/partial_tool_agent_loop.py).

When a weight update aborts the request in flight, the loop returns what it has with ``extra_fields["is_cancel"]``
and its whole conversation state (``extra_fields["agent_data"]``: messages, token / mask / log-prob streams, turn
counters, the tokens of the unfinished assistant turn). Passing that output back (``output=...``) continues the same
assistant turn under the new weights: the tool-call parser sees the turn's tokens from both generations."""

from __future__ import annotations

import time
from typing import Any, Optional

from ...agent_loop.agent_loop import AgentLoopOutput, register
from ...agent_loop.tool_agent_loop import AgentData, AgentState, ToolAgentLoop


@register("partial_tool_agent")
class PartialToolAgentLoop(ToolAgentLoop):
    async def run(self, sampling_params: dict[str, Any], **kwargs) -> AgentLoopOutput:
        prev: Optional[AgentLoopOutput] = kwargs.get("output")
        version = int(kwargs.get("param_version", 0))
        if prev is None:
            out = await super().run(sampling_params, **kwargs)
            start = version
        elif prev.extra_fields.get("is_cancel", False):
            data: AgentData = prev.extra_fields["agent_data"]
            start = prev.extra_fields.get("param_version_start", version)
            out = await self._run_from(data, AgentState.GENERATING, sampling_params)
        else:
            return prev
        out.extra_fields.setdefault("is_cancel", False)
        out.extra_fields.update(param_version_start=start, param_version_end=version)
        return out

    async def _generate(self, data: AgentData, sampling_params: dict) -> AgentState:
        t0 = time.perf_counter()
        sp = dict(sampling_params)
        sp["max_tokens"] = max(self.response_length - len(data.response_ids), 0)
        ids, lps, cancelled = await self.server_manager.generate_for_partial(
            data.request_id, prompt_ids=data.prompt_ids + data.response_ids, sampling_params=sp)
        data.metrics["generate_sequences"] += time.perf_counter() - t0
        return await self._after_generation(data, ids, lps, turn_complete=not cancelled)
