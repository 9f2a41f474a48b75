"""Agent loop: per-sample coroutines that drive generation (and tools) against rollout servers.

Structure of verl/experimental/agent_loop/agent_loop.py: ``AsyncLLMServerManager`` (least-in-flight load
balancing, sticky by request id), ``AgentLoopOutput``, ``AgentLoopBase`` + ``register``, ``AgentLoopWorker``
(runs a chunk of samples concurrently and assembles the padded batch), ``AgentLoopManager`` (chunks a batch
over workers, concatenates, reports timing). Workers are asyncio tasks in this process: the rollout servers
already own the GPUs, the loop itself is CPU-light.
"""

from __future__ import annotations

import asyncio
import heapq
import random
import time
from abc import ABC, abstractmethod
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Any, Optional
from uuid import uuid4

import numpy as np
import torch

from ...protocol import DataProto
from ...rollout import TokenOutput
from ...rollout.postprocess import assemble_rollout_batch

_agent_loop_registry: dict[str, Any] = {}


def register(agent_name: str):
    """Class decorator: make an agent loop selectable by ``agent_name`` (per-sample column or default)."""

    def deco(cls):
        _agent_loop_registry[agent_name] = cls
        return cls

    return deco


class AsyncLLMServerManager:
    """Routes requests to the least-loaded server; a multi-turn conversation sticks to its first server so the
    prefix cache hits (LRU of 10000 request ids, verl/experimental/agent_loop/agent_loop.py:57-122)."""

    def __init__(self, config, server_handles: list, max_cache_size: int = 10000):
        self.config = config
        self.server_handles = list(server_handles)
        random.shuffle(self.server_handles)
        self.load = [[0, i, h] for i, h in enumerate(self.server_handles)]
        heapq.heapify(self.load)
        self.sticky: OrderedDict[str, Any] = OrderedDict()
        self.max_cache_size = max_cache_size

    def _choose_server(self, request_id: str):
        if request_id in self.sticky:
            self.sticky.move_to_end(request_id)
            return self.sticky[request_id]
        entry = self.load[0]
        entry[0] += 1
        heapq.heapreplace(self.load, entry)
        self.sticky[request_id] = entry[2]
        if len(self.sticky) > self.max_cache_size:
            self.sticky.popitem(last=False)
        return entry[2]

    async def generate(self, request_id: str, *, prompt_ids: list[int], sampling_params: dict[str, Any],
                       image_data=None, video_data=None) -> TokenOutput:
        server = self._choose_server(request_id)
        kw = {} if image_data is None and video_data is None else {"image_data": image_data, "video_data": video_data}
        return await server.generate(prompt_ids=prompt_ids, sampling_params=sampling_params, request_id=uuid4().hex, **kw)

    async def generate_for_partial(self, request_id: str, *, prompt_ids: list[int], sampling_params: dict[str, Any],
                                   image_data=None, video_data=None) -> tuple[list[int], list[float], bool]:
        """Generation that may be cut short by ``abort_all_requests`` (a weight update in the fully asynchronous
        pipeline): returns (tokens so far, their log-probs, was_cancelled). The caller resumes a cancelled sample by
        sending prompt + partial response as the next prompt."""
        out = await self.generate(request_id, prompt_ids=prompt_ids, sampling_params=sampling_params)
        return list(out.token_ids), list(out.log_probs or []), out.stop_reason == "aborted"


@dataclass
class AgentLoopMetrics:
    generate_sequences: float = 0.0
    tool_calls: float = 0.0
    num_preempted: int = -1


@dataclass
class AgentLoopOutput:
    prompt_ids: list
    response_ids: list
    response_mask: list  # 1 = model token, 0 = tool / user token
    response_logprobs: Optional[list] = None
    routed_experts: Optional[Any] = None
    multi_modal_data: Optional[dict] = None
    reward_score: Optional[float] = None
    num_turns: int = 0
    metrics: AgentLoopMetrics = field(default_factory=AgentLoopMetrics)
    extra_fields: dict = field(default_factory=dict)


class AgentLoopBase(ABC):
    def __init__(self, trainer_config, server_manager: AsyncLLMServerManager, tokenizer, processor=None, **kwargs):
        self.config = trainer_config
        self.server_manager = server_manager
        self.tokenizer, self.processor = tokenizer, processor
        self.loop = asyncio.get_event_loop()

    async def apply_chat_template(self, messages, tools=None) -> list[int]:
        if isinstance(messages, np.ndarray):
            messages = messages.tolist()
        if len(messages) and isinstance(messages[0], (int, np.integer)):
            return [int(t) for t in messages]
        kw = {"tools": tools} if tools else {}
        return list(await self.loop.run_in_executor(
            None, lambda: self.tokenizer.apply_chat_template(messages, add_generation_prompt=True, tokenize=True, **kw)))

    @abstractmethod
    async def run(self, sampling_params: dict[str, Any], **kwargs) -> AgentLoopOutput:
        ...


class AgentLoopWorker:
    """Runs the agent loops of a chunk of samples concurrently and pads the results into a batch."""

    def __init__(self, config, server_handles: list, tokenizer, processor=None, reward_fn=None):
        self.config = config
        self.server_manager = AsyncLLMServerManager(config, server_handles)
        self.tokenizer, self.processor = tokenizer, processor
        self.reward_fn = reward_fn
        from . import single_turn_agent_loop, tool_agent_loop  # noqa: F401  (registers the built-in loops)

        agent = config.actor_rollout_ref.rollout.agent
        path = agent.get("agent_loop_config_path", None) if hasattr(agent, "get") else getattr(agent, "agent_loop_config_path", None)
        if path:
            # a YAML list of ``{name, _target_: package.module.Class, **constructor arguments}``: user-defined loops
            import importlib
            import os

            import yaml

            for entry in yaml.safe_load(open(os.path.expanduser(str(path)))) or []:
                entry = dict(entry)
                name, target = entry.pop("name"), entry.pop("_target_")
                mod, _, cls = str(target).rpartition(".")
                _agent_loop_registry[name] = (getattr(importlib.import_module(mod), cls), entry)
        model = config.actor_rollout_ref.model
        template = model.get("custom_chat_template", None) if hasattr(model, "get") else getattr(model, "custom_chat_template", None)
        if template is not None:
            for obj in (self.tokenizer, self.processor):
                if obj is not None:
                    obj.chat_template = template

    async def generate_sequences(self, batch: DataProto) -> DataProto:
        rc = self.config.actor_rollout_ref.rollout
        sp = dict(temperature=rc.temperature, top_p=rc.top_p, top_k=rc.top_k, repetition_penalty=1.0,
                  logprobs=rc.get("calculate_log_probs", False) or True)
        if batch.meta_info.get("validate", False):
            vk = rc.val_kwargs
            sp.update(temperature=vk.temperature if vk.do_sample else 0.0, top_p=vk.top_p, top_k=vk.top_k)
        n = len(batch)
        default = rc.agent.get("default_agent_loop", "single_turn_agent")
        names = batch.non_tensor_batch.get("agent_name", np.array([default] * n, dtype=object))
        tasks = []
        for i in range(n):
            kwargs = {k: v[i] for k, v in batch.non_tensor_batch.items() if k != "agent_name"}
            if "raw_prompt" not in kwargs and "raw_prompt_ids" in kwargs:
                kwargs["raw_prompt"] = kwargs["raw_prompt_ids"]
            tasks.append(asyncio.create_task(self._run_agent_loop(str(names[i] or default), dict(sp), **kwargs)))
        outputs: list[AgentLoopOutput] = await asyncio.gather(*tasks)
        return self._postprocess(outputs, rc)

    async def _run_agent_loop(self, agent_name: str, sampling_params: dict, **kwargs) -> AgentLoopOutput:
        assert agent_name in _agent_loop_registry, f"Agent loop {agent_name} not registered, registered agent loops: {list(_agent_loop_registry)}"
        entry = _agent_loop_registry[agent_name]
        cls, extra = entry if isinstance(entry, tuple) else (entry, {})
        loop = cls(trainer_config=self.config, server_manager=self.server_manager, tokenizer=self.tokenizer,
                   processor=self.processor, **extra)
        return await loop.run(sampling_params, **kwargs)

    def _postprocess(self, outputs: list[AgentLoopOutput], rc) -> DataProto:
        P, R = int(rc.prompt_length), int(rc.response_length)
        pad = getattr(self.tokenizer, "pad_token_id", 0) or 0
        B = len(outputs)
        prompts = torch.full((B, P), pad, dtype=torch.long)
        pmask = torch.zeros(B, P, dtype=torch.long)
        shells = []
        for i, o in enumerate(outputs):
            p = list(o.prompt_ids)[-P:]
            prompts[i, P - len(p):] = torch.tensor(p, dtype=torch.long)
            pmask[i, P - len(p):] = 1
            rec = o.routed_experts
            if rec is not None:
                # the record of ONE generation call covers its prompt and its response; cut it like the prompt
                rec = rec[len(o.prompt_ids) - len(p):] if len(rec) == len(o.prompt_ids) + len(o.response_ids) else None
            shells.append(TokenOutput(token_ids=list(o.response_ids)[:R], log_probs=o.response_logprobs, routed_experts=rec))
        has_lp = all(o.response_logprobs is not None for o in outputs)
        out = assemble_rollout_batch(prompts, pmask, shells, R, pad, with_logprobs=has_lp,
                                     response_masks=[o.response_mask for o in outputs])
        mms = [(o.multi_modal_data or {}).get("multi_modal_inputs") for o in outputs]
        if self.processor is not None and any(m is not None for m in mms):
            # vision-language samples: [B, 4, S] position ids (text positions + multimodal RoPE of prompt and response)
            from ...utils.dataset.vision_utils import vl_position_ids

            out.batch["position_ids"] = vl_position_ids(out.batch["input_ids"], out.batch["attention_mask"], mms,
                                                        self.processor.image_token_id, self.processor.merge_size,
                                                        video_token_id=getattr(self.processor, "video_token_id", None))
        scores = [o.reward_score for o in outputs]
        if all(s is not None for s in scores):
            rm = torch.zeros(B, R)
            lens = out.batch["attention_mask"][:, P:].sum(-1).clamp(min=1)
            rm[torch.arange(B), lens - 1] = torch.tensor(scores, dtype=torch.float32)
            out.batch["rm_scores"] = rm
        out.non_tensor_batch["__num_turns__"] = np.array([o.num_turns for o in outputs], dtype=np.int32)
        extra_keys = sorted({k for o in outputs for k in o.extra_fields})
        for k in extra_keys:
            arr = np.empty(B, dtype=object)
            arr[:] = [o.extra_fields.get(k) for o in outputs]
            out.non_tensor_batch[k] = arr
        out.meta_info["metrics"] = [{"generate_sequences": o.metrics.generate_sequences, "tool_calls": o.metrics.tool_calls,
                                     "num_preempted": o.metrics.num_preempted} for o in outputs]
        out.meta_info["reward_extra_keys"] = []
        return out


class AgentLoopManager:
    """Owns the rollout replicas' server handles and a pool of agent-loop workers."""

    def __init__(self, config, worker_group=None, server_handles: Optional[list] = None, tokenizer=None, processor=None,
                 replicas: Optional[list] = None):
        self.config = config
        self.worker_group = worker_group
        self.rollout_replicas = replicas or []
        self.server_handles = list(server_handles or [r.server_handle for r in self.rollout_replicas])
        self.server_addresses = [getattr(r, "server_address", None) for r in self.rollout_replicas]
        n = int(config.actor_rollout_ref.rollout.agent.get("num_workers", 1))
        self.agent_loop_workers = [AgentLoopWorker(config, self.server_handles, tokenizer, processor) for _ in range(max(n, 1))]

    async def generate_sequences_async(self, prompts: DataProto) -> DataProto:
        t0 = time.perf_counter()
        n = min(len(self.agent_loop_workers), max(len(prompts), 1))
        sizes = [len(prompts) // n + (1 if i < len(prompts) % n else 0) for i in range(n)]
        chunks, s = [], 0
        for sz in sizes:
            chunks.append(prompts[s : s + sz])
            s += sz
        outs = await asyncio.gather(*[w.generate_sequences(c) for w, c in zip(self.agent_loop_workers, chunks) if len(c)])
        metrics = [m for o in outs for m in o.meta_info.pop("metrics", [])]
        for o in outs:
            o.meta_info.pop("reward_extra_keys", None)
        out = DataProto.concat(outs)
        out.meta_info["timing"] = self._performance_metrics(metrics, out, time.perf_counter() - t0)
        return out

    def generate_sequences(self, prompts: DataProto) -> DataProto:
        try:
            loop = asyncio.get_running_loop()
        except RuntimeError:
            loop = None
        if loop is None:
            return asyncio.run(self.generate_sequences_async(prompts))
        raise RuntimeError("call generate_sequences_async() from inside an event loop")

    def _performance_metrics(self, metrics: list[dict], output: DataProto, wall: float) -> dict[str, float]:
        timing = {"agent_loop/wall": wall}
        if not metrics:
            return timing
        gen = np.array([m["generate_sequences"] for m in metrics])
        tool = np.array([m["tool_calls"] for m in metrics])
        pre = np.array([m["num_preempted"] for m in metrics])
        timing.update({"agent_loop/generate_sequences/min": float(gen.min()), "agent_loop/generate_sequences/max": float(gen.max()),
                       "agent_loop/generate_sequences/mean": float(gen.mean()), "agent_loop/tool_calls/min": float(tool.min()),
                       "agent_loop/tool_calls/max": float(tool.max()), "agent_loop/tool_calls/mean": float(tool.mean()),
                       "agent_loop/num_preempted/max": float(pre.max()), "agent_loop/num_preempted/mean": float(pre.mean())})
        slow = int(np.argmax(gen + tool))
        mask = output.batch["attention_mask"][slow]
        P = output.batch["prompts"].shape[1]
        timing.update({"agent_loop/slowest/generate_sequences": float(gen[slow]), "agent_loop/slowest/tool_calls": float(tool[slow]),
                       "agent_loop/slowest/prompt_length": float(mask[:P].sum()), "agent_loop/slowest/response_length": float(mask[P:].sum())})
        return timing

    def wake_up(self):
        for r in self.rollout_replicas:
            asyncio.run(r.wake_up())

    def sleep(self):
        for r in self.rollout_replicas:
            asyncio.run(r.sleep())

    def _run_all(self, coros: list) -> list:
        async def run_all():
            return await asyncio.gather(*coros)

        return asyncio.run(run_all()) if coros else []

    def _targets(self) -> list:
        """The replicas when there are any, else the server handles themselves (the colocated layout)."""
        return list(self.rollout_replicas) or list(self.server_handles)

    def clear_kv_cache(self):
        """Drop all cached keys / values (prefix cache included) of every replica without putting it to sleep."""
        self._run_all([t.clear_kv_cache() for t in self._targets() if hasattr(t, "clear_kv_cache")])

    def start_profile(self, **kwargs):
        self._run_all([t.start_profile(**kwargs) for t in self._targets() if hasattr(t, "start_profile")])

    def stop_profile(self):
        self._run_all([t.stop_profile() for t in self._targets() if hasattr(t, "stop_profile")])


async def get_trajectory_info(step: int, index: list, validate: bool) -> list[dict]:
    """One record per sample for rollout traces: the trainer step, the dataset index of the sample's prompt and the
    number of the sample among the consecutive samples of the same prompt."""
    out, n = [], 0
    for i, idx in enumerate(index):
        n = n + 1 if i > 0 and index[i - 1] == idx else 0
        out.append({"step": step, "sample_index": idx, "rollout_n": n, "validate": validate})
    return out
