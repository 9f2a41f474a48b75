"""Multi-turn tool-calling agent loop.

State machine of verl/experimental/agent_loop/tool_agent_loop.py:46-190:
``PENDING -> GENERATING -> PROCESSING_TOOLS -> (INTERACTING) -> GENERATING ... -> TERMINATED``.
Model tokens get response_mask 1, tool / user tokens (appended as a tokenised chat turn) get 0; generation stops
at the response-length budget, the assistant / user turn limits, or when the model emits no tool call.
"""

from __future__ import annotations

import asyncio
import json
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Optional
from uuid import uuid4

from ...tools.schemas import OpenAIFunctionCallSchema, OpenAIFunctionParsedSchema, ToolResponse
from .agent_loop import AgentLoopBase, AgentLoopMetrics, AgentLoopOutput, register
from .tool_parser import FunctionCall, ToolParser


class AgentState(Enum):
    PENDING = "pending"
    GENERATING = "generating"
    PROCESSING_TOOLS = "processing_tools"
    INTERACTING = "interacting"
    TERMINATED = "terminated"
    CANCELLED = "cancelled"  # generation aborted by a weight update: resumable (partial rollout)


@dataclass
class AgentData:
    messages: list
    tools_kwargs: dict
    interaction_kwargs: dict
    request_id: str
    prompt_ids: list = field(default_factory=list)
    response_ids: list = field(default_factory=list)
    response_mask: list = field(default_factory=list)
    response_logprobs: list = field(default_factory=list)
    turn_ids: list = field(default_factory=list)  # ids generated in the current assistant turn
    tool_calls: list = field(default_factory=list)
    tool_rewards: list = field(default_factory=list)
    turn_scores: list = field(default_factory=list)
    user_turns: int = 0
    assistant_turns: int = 0
    metrics: dict = field(default_factory=lambda: {"generate_sequences": 0.0, "tool_calls": 0.0, "num_preempted": 0})
    interaction: Any = None
    mid_turn: bool = False  # the current assistant turn was cut by an abort and continues in the next generation
    routed_experts: Any = None  # mixture-of-experts rollouts that record their routing: the latest call's record


_TOOLS_CACHE: dict = {}
_INTERACTIONS_CACHE: dict = {}


@register("tool_agent")
class ToolAgentLoop(AgentLoopBase):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        rc = self.config.actor_rollout_ref.rollout
        mt = rc.multi_turn
        self.max_user_turns = mt.get("max_user_turns")
        self.max_assistant_turns = mt.get("max_assistant_turns")
        self.max_parallel_calls = int(mt.get("max_parallel_calls", 1))
        self.max_tool_response_length = int(mt.get("max_tool_response_length", 256))
        self.truncate_side = mt.get("tool_response_truncate_side", "middle")
        self.prompt_length, self.response_length = int(rc.prompt_length), int(rc.response_length)
        path = mt.get("tool_config_path")
        if path and path not in _TOOLS_CACHE:
            from ...tools.utils.tool_registry import initialize_tools_from_config

            _TOOLS_CACHE[path] = initialize_tools_from_config(path)
        tool_list = _TOOLS_CACHE.get(path, []) if path else []
        self.tools = {t.name: t for t in tool_list}
        self.tool_schemas = [t.tool_schema.model_dump(exclude_unset=True, exclude_none=True) for t in tool_list]
        self.tool_parser = ToolParser.get_tool_parser(mt.get("format", "hermes"), self.tokenizer)
        ipath = mt.get("interaction_config_path")
        if ipath and ipath not in _INTERACTIONS_CACHE:
            from ...interactions.utils.interaction_registry import initialize_interactions_from_config

            _INTERACTIONS_CACHE[ipath] = initialize_interactions_from_config(ipath)
        self.interactions = _INTERACTIONS_CACHE.get(ipath, {}) if ipath else {}

    async def run(self, sampling_params: dict[str, Any], **kwargs) -> AgentLoopOutput:
        messages = kwargs["raw_prompt"]
        messages = messages.tolist() if hasattr(messages, "tolist") else list(messages)
        data = AgentData(messages=messages, tools_kwargs=kwargs.get("tools_kwargs") or {},
                         interaction_kwargs=kwargs.get("interaction_kwargs") or {}, request_id=uuid4().hex)
        if self.interactions and data.interaction_kwargs:
            name = data.interaction_kwargs.get("name") or next(iter(self.interactions))
            if name not in self.interactions:
                raise ValueError(f"Interaction '{name}' not found in interaction_map. Available interactions: {list(self.interactions)}")
            data.interaction = self.interactions[name]
            await data.interaction.start_interaction(data.request_id, **data.interaction_kwargs)
        return await self._run_from(data, AgentState.PENDING, sampling_params)

    async def _run_from(self, data: AgentData, state: AgentState, sampling_params: dict[str, Any]) -> AgentLoopOutput:
        """Drive the state machine from ``state`` until it terminates (or is cancelled: see the partial-rollout
        subclass in ``fully_async_policy/agent_loop``)."""
        while state not in (AgentState.TERMINATED, AgentState.CANCELLED):
            if state == AgentState.PENDING:
                data.prompt_ids = await self.apply_chat_template(data.messages, tools=self.tool_schemas or None)
                state = AgentState.GENERATING
            elif state == AgentState.GENERATING:
                state = await self._generate(data, sampling_params)
            elif state == AgentState.PROCESSING_TOOLS:
                state = await self._process_tools(data)
            elif state == AgentState.INTERACTING:
                state = await self._interact(data)
        return self._output(data, cancelled=state == AgentState.CANCELLED)

    def _output(self, data: AgentData, cancelled: bool = False) -> AgentLoopOutput:
        ids = data.response_ids[: self.response_length]
        extra = {"turn_scores": data.turn_scores, "tool_rewards": data.tool_rewards}
        if cancelled:
            extra.update(is_cancel=True, agent_data=data)
        routed = data.routed_experts
        if routed is not None:
            # tokens appended after the last call (a final tool response) were never routed: zero rows, like padding
            import numpy as np

            total = len(data.prompt_ids) + len(ids)
            full = np.zeros((total,) + tuple(routed.shape[1:]), routed.dtype)
            full[: min(total, routed.shape[0])] = routed[:total]
            routed = full
        return AgentLoopOutput(
            prompt_ids=data.prompt_ids, response_ids=ids, response_mask=data.response_mask[: self.response_length],
            response_logprobs=data.response_logprobs[: self.response_length] if data.response_logprobs else None,
            routed_experts=routed, num_turns=data.user_turns + data.assistant_turns + 1,
            metrics=AgentLoopMetrics(**data.metrics), extra_fields=extra)

    # ------------------------------------------------------------------ states
    async def _generate(self, data: AgentData, sampling_params: dict) -> AgentState:
        t0 = time.perf_counter()
        ctx = data.prompt_ids + data.response_ids
        sp = dict(sampling_params)
        sp["max_tokens"] = max(self.response_length - len(data.response_ids), 0)
        out = await self.server_manager.generate(data.request_id, prompt_ids=ctx, sampling_params=sp)
        data.metrics["generate_sequences"] += time.perf_counter() - t0
        data.metrics["num_preempted"] += max(out.num_preempted, 0)
        if out.routed_experts is not None:
            # router replay R3: the record of a call covers its whole context (prompt, earlier turns, tool responses)
            # and its own tokens, so the latest call's record is the record of the sequence so far
            data.routed_experts = out.routed_experts
        return await self._after_generation(data, list(out.token_ids), list(out.log_probs or []))

    async def _after_generation(self, data: AgentData, token_ids: list, log_probs: list, turn_complete: bool = True) -> AgentState:
        """Book the tokens of an assistant turn (``turn_complete=False``: the turn was cut and will be continued)."""
        if not data.mid_turn:
            data.assistant_turns += 1
            data.turn_ids = []
        data.turn_ids += token_ids
        data.response_ids += token_ids
        data.response_mask += [1] * len(token_ids)
        if log_probs:
            data.response_logprobs += log_probs
        data.mid_turn = not turn_complete
        if len(data.response_ids) >= self.response_length:
            data.mid_turn = False
            return AgentState.TERMINATED
        if not turn_complete:
            return AgentState.CANCELLED
        if self.max_assistant_turns and data.assistant_turns >= self.max_assistant_turns:
            return AgentState.TERMINATED
        if self.max_user_turns and data.user_turns >= self.max_user_turns:
            return AgentState.TERMINATED
        _, data.tool_calls = await self.tool_parser.extract_tool_calls(data.turn_ids)
        if data.tool_calls and self.tools:
            return AgentState.PROCESSING_TOOLS
        if data.interaction is not None:
            text = self.tokenizer.decode(data.turn_ids, skip_special_tokens=True)
            data.messages.append({"role": "assistant", "content": text})
            return AgentState.INTERACTING
        return AgentState.TERMINATED

    async def _append_turn(self, data: AgentData, new_messages: list[dict]) -> bool:
        """Tokenise extra chat turns (without the system prefix) and append them with mask 0."""
        ids = await self.loop.run_in_executor(None, lambda: self._encode_turns(new_messages))
        if len(data.response_ids) + len(ids) >= self.response_length:
            return False
        data.response_ids += ids
        data.response_mask += [0] * len(ids)
        if data.response_logprobs:
            data.response_logprobs += [0.0] * len(ids)
        data.user_turns += 1
        return True

    def _encode_turns(self, msgs: list[dict]) -> list[int]:
        tok = self.tokenizer
        full = tok.apply_chat_template([{"role": "user", "content": ""}] + msgs, add_generation_prompt=True, tokenize=True)
        base = tok.apply_chat_template([{"role": "user", "content": ""}], add_generation_prompt=False, tokenize=True)
        full, base = list(full), list(base)
        return full[len(base):] if full[: len(base)] == base else full

    async def _process_tools(self, data: AgentData) -> AgentState:
        t0 = time.perf_counter()
        calls = data.tool_calls[: self.max_parallel_calls]
        results = await asyncio.gather(*[self._call_tool(c, data.tools_kwargs) for c in calls])
        data.metrics["tool_calls"] += time.perf_counter() - t0
        msgs = []
        for resp, reward in results:
            msgs.append({"role": "tool", "content": resp.text or ""})
            if reward is not None:
                data.tool_rewards.append(reward)
        data.messages.extend(msgs)
        if not await self._append_turn(data, msgs):
            return AgentState.TERMINATED
        return AgentState.GENERATING

    async def _call_tool(self, call: FunctionCall, tools_kwargs: dict) -> tuple[ToolResponse, Optional[float]]:
        tool, instance_id = None, None
        try:
            parsed, bad = OpenAIFunctionCallSchema.from_openai_function_parsed_schema(
                OpenAIFunctionParsedSchema(name=call.name, arguments=call.arguments))
            if call.name not in self.tools:
                return ToolResponse(text=f"Error when executing tool: unknown tool {call.name}"), None
            tool = self.tools[call.name]
            kw = tools_kwargs.get(call.name, {}) if isinstance(tools_kwargs, dict) else {}
            instance_id, _ = await tool.create(create_kwargs=kw.get("create_kwargs", {}), **kw.get("create_kwargs", {}))
            resp, reward, _ = await tool.execute(instance_id, parsed.arguments, **kw.get("execute_kwargs", {}))
        except Exception as e:
            return ToolResponse(text=f"Error when executing tool: {e}"), None
        finally:
            if tool is not None and instance_id is not None:
                await tool.release(instance_id)
        text = resp.text or ""
        L = self.max_tool_response_length
        if len(text) > L:
            if self.truncate_side == "left":
                text = text[:L] + "...(truncated)"
            elif self.truncate_side == "right":
                text = "(truncated)..." + text[-L:]
            else:
                text = text[: L // 2] + "...(truncated)..." + text[-(L // 2):]
        return ToolResponse(text=text, image=resp.image, video=resp.video), reward

    async def _interact(self, data: AgentData) -> AgentState:
        stop, text, score, _ = await data.interaction.generate_response(data.request_id, data.messages, **data.interaction_kwargs)
        data.turn_scores.append(score)
        if stop:
            return AgentState.TERMINATED
        msg = [{"role": "user", "content": text}]
        data.messages.extend(msg)
        if not await self._append_turn(data, msg):
            return AgentState.TERMINATED
        return AgentState.GENERATING
