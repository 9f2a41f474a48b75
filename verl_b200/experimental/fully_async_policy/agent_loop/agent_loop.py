"""Agent-loop workers for the fully asynchronous pipeline: samples whose generation is cut by a weight update are
handed back un-padded, kept by the caller and continued later
(verl/experimental/fully_async_policy/agent_loop/agent_loop.py: ``FullyAsyncLLMServerManager``,
``FullyAsyncAgentLoopWorker``, ``FullyAsyncAgentLoopManager``).

Flow of one prompt group (``n`` samples of one prompt):

    outs, cancelled = await manager.generate_single_sample_async(group, None, version)
    while cancelled:                       # a parameter update aborted the requests in flight
        await manager.wait_resumed()
        outs, cancelled = await manager.generate_single_sample_async(group, outs, new_version)
    batch = manager.postprocess(outs)      # padded DataProto, as the synchronous manager returns

``cancel()`` aborts every request on every server (the engines return the tokens generated so far) and blocks new
generations until ``resume()``.
"""

from __future__ import annotations

import asyncio
from typing import Optional

import numpy as np

from ....protocol import DataProto
from ...agent_loop.agent_loop import AgentLoopManager, AgentLoopOutput, AgentLoopWorker, AsyncLLMServerManager

_PARTIAL_NAME = {"single_turn_agent": "partial_single_turn_agent", "tool_agent": "partial_tool_agent"}


class FullyAsyncLLMServerManager(AsyncLLMServerManager):
    """Load-balancing server manager; ``generate_for_partial`` (inherited) reports whether a generation was cut."""


class FullyAsyncAgentLoopWorker(AgentLoopWorker):
    def __init__(self, config, server_handles: list, tokenizer, processor=None, reward_fn=None):
        super().__init__(config, server_handles, tokenizer, processor, reward_fn)
        self.server_manager = FullyAsyncLLMServerManager(config, server_handles)
        from . import partial_single_turn_agent_loop, partial_tool_agent_loop  # noqa: F401  (registers the loops)

    def _sampling(self, batch: DataProto) -> dict:
        rc = self.config.actor_rollout_ref.rollout
        sp = dict(temperature=rc.temperature, top_p=rc.top_p, top_k=rc.top_k, repetition_penalty=1.0, logprobs=True)
        if batch.meta_info.get("validate", False):
            vk = rc.val_kwargs
            sp.update(temperature=vk.temperature if vk.do_sample else 0.0, top_p=vk.top_p, top_k=vk.top_k)
        return sp

    async def generate_sequences_no_post(self, batch: DataProto, partial_output_list: Optional[list[AgentLoopOutput]],
                                         param_version: int = 0) -> list[AgentLoopOutput]:
        """One agent loop per row; rows that already finished (``partial_output_list[i]`` not cancelled) come back
        unchanged, cancelled ones continue, ``None`` starts fresh. Nothing is padded."""
        rc = self.config.actor_rollout_ref.rollout
        sp = self._sampling(batch)
        n = len(batch)
        default = rc.agent.get("default_agent_loop", "single_turn_agent")
        names = batch.non_tensor_batch.get("agent_name", np.array([default] * n, dtype=object))
        prev = partial_output_list or [None] * n
        tasks = []
        for i in range(n):
            kwargs = {k: v[i] for k, v in batch.non_tensor_batch.items()}
            if "raw_prompt" not in kwargs and "raw_prompt_ids" in kwargs:
                kwargs["raw_prompt"] = kwargs["raw_prompt_ids"]
            kwargs.update(output=prev[i], param_version=param_version)
            name = str(names[i] or default)
            tasks.append(asyncio.create_task(self._run_agent_loop(_PARTIAL_NAME.get(name, name), dict(sp), **kwargs)))
        return list(await asyncio.gather(*tasks))

    def postprocess(self, outputs: list[AgentLoopOutput]) -> DataProto:
        for o in outputs:
            o.extra_fields.pop("agent_data", None)  # conversation state of a resumable loop: not batch data
        out = self._postprocess(outputs, self.config.actor_rollout_ref.rollout)
        out.meta_info.pop("reward_extra_keys", None)
        return out


class FullyAsyncAgentLoopManager(AgentLoopManager):
    def __init__(self, config, worker_group=None, server_handles: Optional[list] = None, tokenizer=None, processor=None,
                 replicas: Optional[list] = None):
        super().__init__(config, worker_group, server_handles, tokenizer, processor, replicas)
        self.agent_loop_workers = [FullyAsyncAgentLoopWorker(config, self.server_handles, tokenizer, processor)
                                   for _ in range(len(self.agent_loop_workers))]
        self._next = 0
        self._running: Optional[asyncio.Event] = None

    def _gate(self) -> asyncio.Event:
        if self._running is None:
            self._running = asyncio.Event()
            self._running.set()
        return self._running

    async def generate_single_sample_async(self, sample: DataProto, partial_output_list: Optional[list[AgentLoopOutput]],
                                           param_version: int = 0) -> tuple[list[AgentLoopOutput], bool]:
        """Returns (outputs, any_cancelled)."""
        await self._gate().wait()
        w = self.agent_loop_workers[self._next % len(self.agent_loop_workers)]
        self._next += 1
        outs = await w.generate_sequences_no_post(sample, partial_output_list, param_version)
        return outs, any(o.extra_fields.get("is_cancel", False) for o in outs)

    def postprocess(self, outputs: list[AgentLoopOutput]) -> DataProto:
        return self.agent_loop_workers[0].postprocess(outputs)

    async def cancel(self) -> None:
        """Abort the requests in flight on every server and hold new generations back until :meth:`resume`."""
        self._gate().clear()
        await asyncio.gather(*[h.abort_all_requests(reset_prefix_cache=False) for h in self.server_handles])

    async def resume(self) -> None:
        await asyncio.gather(*[h.resume_all_requests() for h in self.server_handles])
        self._gate().set()

    async def wait_resumed(self) -> None:
        await self._gate().wait()

    async def clear_kv_cache(self) -> None:
        await asyncio.gather(*[h.clear_kv_cache() for h in self.server_handles])
