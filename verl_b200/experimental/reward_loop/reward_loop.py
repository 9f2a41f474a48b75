"""Reward loop: asynchronous reward computation next to (and overlapped with) generation.

Role of verl/experimental/reward_loop/reward_loop.py:40-330: ``RewardLoopWorker`` scores samples one by one with a
reward manager (rule-based, custom function, or a reward model behind a router); ``RewardLoopManager`` owns the
workers, splits a batch across them and assembles ``rm_scores`` (score on the last valid response token) plus the
``reward_extra_info`` columns. The reference runs the workers as Ray actors; here they are asyncio workers of one
event loop thread (scoring functions run in executor threads / processes), which keeps the same concurrency model
without an RPC layer.
"""

from __future__ import annotations

import asyncio
import threading
from collections import defaultdict
from typing import Optional

import numpy as np
import torch

from ...protocol import DataProto
from ...trainer.ppo.reward import get_custom_reward_fn
from .reward_manager import get_reward_manager_cls


class RewardLoopWorker:
    def __init__(self, config, tokenizer, reward_router_address: Optional[str] = None, reward_model_tokenizer=None,
                 reward_model_manager=None):
        self.config = config
        self.tokenizer = tokenizer
        self.reward_router_address = reward_router_address
        self.reward_model_manager = reward_model_manager
        rm = config.get("reward_model") or {}
        source = rm.get("reward_loop_source", "register")
        if source == "register":
            cls = get_reward_manager_cls(rm.get("reward_manager", "naive"))
        elif source == "importlib":
            from ...utils.py_functional import load_extern_object

            assert rm.get("reward_loop_module_path") and rm.get("reward_loop_class_name"), \
                "reward_loop_module_path / reward_loop_class_name must be set when reward_loop_source='importlib'"
            cls = load_extern_object(rm["reward_loop_module_path"], rm["reward_loop_class_name"])
        else:
            raise ValueError(f"Unknown reward_loop_source: {source}. Must be 'register' or 'importlib'")
        self.custom_fn = get_custom_reward_fn(config)
        self.reward_loop = cls(config, tokenizer, self.custom_fn, reward_router_address, reward_model_tokenizer)

    async def compute_score_batch(self, data: DataProto) -> list[dict]:
        return list(await asyncio.gather(*[self.compute_score(data[i : i + 1]) for i in range(len(data))]))

    async def compute_score(self, data: DataProto) -> dict:
        assert len(data) == 1, "RewardLoopWorker scores one sample at a time"
        rm = self.config.get("reward_model") or {}
        if self.custom_fn is None and rm.get("enable", False) and self.reward_model_manager is not None:
            # discriminative reward model; a generative one needs a custom reward function that calls the router
            return await self.compute_score_disrm(data)
        return await self.reward_loop.run_single(data)

    async def compute_score_disrm(self, data: DataProto) -> dict:
        """Score of a discriminative reward model (a value head on the last valid token) for one sample; the manager
        batches concurrent requests into one forward."""
        assert self.reward_model_manager is not None, "no reward model manager was given to this worker"
        score = await self.reward_model_manager.score(data)
        return {"reward_score": float(score), "reward_extra_info": {}}


class RewardLoopManager:
    """Batch front end: ``compute_rm_score(data)`` -> DataProto with ``rm_scores`` [B, R] and extra-info columns."""

    def __init__(self, config, tokenizer, num_workers: Optional[int] = None, reward_model_manager=None,
                 reward_router_address: Optional[str] = None):
        rm = config.get("reward_model") or {}
        n = int(num_workers or rm.get("num_workers", 1) or 1)
        self.workers = [RewardLoopWorker(config, tokenizer, reward_router_address, None, reward_model_manager) for _ in range(n)]
        self._loop = asyncio.new_event_loop()
        self._thread = threading.Thread(target=self._loop.run_forever, name="reward-loop", daemon=True)
        self._thread.start()

    def _run(self, coro):
        return asyncio.run_coroutine_threadsafe(coro, self._loop)

    def compute_rm_score_async(self, data: DataProto):
        """Start scoring; returns a future whose result is the DataProto (lets the trainer overlap it with log-probs)."""
        chunks = [c for c in data.chunk(len(self.workers))] if len(data) % len(self.workers) == 0 else self._uneven(data)

        async def go():
            parts = await asyncio.gather(*[w.compute_score_batch(c) for w, c in zip(self.workers, chunks) if len(c)])
            return [r for p in parts for r in p]

        fut = self._run(go())
        return _Mapped(fut, lambda results: self._assemble(data, results))

    def compute_rm_score(self, data: DataProto) -> DataProto:
        return self.compute_rm_score_async(data).result()

    def _uneven(self, data: DataProto) -> list[DataProto]:
        n, w = len(data), len(self.workers)
        bounds = np.linspace(0, n, w + 1).astype(int)
        return [data[int(a) : int(b)] for a, b in zip(bounds[:-1], bounds[1:])]

    @staticmethod
    def _assemble(data: DataProto, results: list[dict]) -> DataProto:
        R = data.batch["responses"].shape[-1]
        valid = data.batch["attention_mask"][:, -R:].sum(-1).long()
        scores = torch.zeros(len(data), R, dtype=torch.float32)
        extra = defaultdict(list)
        keys = sorted({k for r in results for k in r.get("reward_extra_info", {})})
        for i, r in enumerate(results):
            if valid[i] > 0:
                scores[i, valid[i] - 1] = float(r["reward_score"])
            for k in keys:
                extra[k].append(r.get("reward_extra_info", {}).get(k))
        nt = {}
        for k, v in extra.items():
            arr = np.empty(len(v), dtype=object)
            arr[:] = v
            nt[k] = arr
        return DataProto.from_dict(tensors={"rm_scores": scores}, non_tensors=nt, meta_info={"reward_extra_keys": keys})

    def shutdown(self):
        self._loop.call_soon_threadsafe(self._loop.stop)
        self._thread.join(timeout=5)


class _Mapped:
    def __init__(self, fut, fn):
        self._fut, self._fn = fut, fn

    def result(self, timeout=None):
        return self._fn(self._fut.result(timeout))

    def done(self):
        return self._fut.done()
