"""Asynchronous reward managers (one sample at a time, many in flight).

Role of verl/experimental/reward_loop/reward_manager/{base,registry,naive,dapo,limited,remote}.py: a manager turns
one decoded (prompt, response) into ``{"reward_score": float, "reward_extra_info": {...}}``; sync scoring functions
run in the event loop's executor, async ones are awaited. ``rate_limited`` adds three limiters shared by every
instance in the process (concurrency, requests / minute, tokens / minute) for judge APIs.
"""

from __future__ import annotations

import asyncio
import inspect
import logging
from typing import Any, Callable, Optional

from ...protocol import DataProto
from ...utils.reward_score import default_compute_score

logger = logging.getLogger(__name__)

_REGISTRY: dict[str, type] = {}


def register(name: str):
    def deco(cls):
        if name in _REGISTRY and _REGISTRY[name] is not cls:
            raise ValueError(f"reward loop manager {name!r} is already registered to {_REGISTRY[name]}")
        _REGISTRY[name] = cls
        return cls

    return deco


def get_reward_manager_cls(name: str) -> type:
    if name not in _REGISTRY:
        raise ValueError(f"Unknown reward manager: {name}. Known: {sorted(_REGISTRY)}")
    return _REGISTRY[name]


def _rm_cfg(config) -> dict:
    rm = (config.get("reward_model") if hasattr(config, "get") else None) or {}
    return rm


class RewardManagerBase:
    """``run_single(data)`` scores a DataProto of length 1."""

    def __init__(self, config, tokenizer, compute_score: Optional[Callable] = None, reward_router_address: Optional[str] = None,
                 reward_model_tokenizer=None):
        self.config, self.tokenizer = config, tokenizer
        self.compute_score = compute_score or default_compute_score
        self.is_async = inspect.iscoroutinefunction(self.compute_score)
        self.reward_router_address = reward_router_address
        self.reward_model_tokenizer = reward_model_tokenizer

    # ------------------------------------------------------------------ helpers
    def _decode(self, data: DataProto) -> tuple[str, str, int]:
        item = data[0]
        resp_ids = item.batch["responses"]
        L = resp_ids.shape[-1]
        mask = item.batch["attention_mask"]
        valid = int(mask[-L:].sum())
        prompt_len = int(mask[:-L].sum())
        prompt_ids = item.batch["prompts"][-prompt_len:] if "prompts" in item.batch.keys() and prompt_len else resp_ids[:0]
        prompt = self.tokenizer.decode(prompt_ids.tolist(), skip_special_tokens=True)
        response = self.tokenizer.decode(resp_ids[:valid].tolist(), skip_special_tokens=True)
        return prompt, response, valid

    async def _score(self, **kw) -> Any:
        if self.reward_router_address is not None and "reward_router_address" in inspect.signature(self.compute_score).parameters:
            kw["reward_router_address"] = self.reward_router_address
            kw["reward_model_tokenizer"] = self.reward_model_tokenizer
        if self.is_async:
            return await self.compute_score(**kw)
        loop = asyncio.get_running_loop()
        return await loop.run_in_executor(None, lambda: self.compute_score(**kw))

    @staticmethod
    def _pack(result) -> dict:
        if isinstance(result, dict):
            score = float(result["score"])
            return {"reward_score": score, "reward_extra_info": {k: v for k, v in result.items()}}
        return {"reward_score": float(result), "reward_extra_info": {"acc": float(result)}}

    async def run_single(self, data: DataProto) -> dict:
        raise NotImplementedError


@register("naive")
class NaiveRewardManager(RewardManagerBase):
    async def run_single(self, data: DataProto) -> dict:
        assert len(data) == 1, "one sample at a time"
        _, response, _ = self._decode(data)
        nt = data[0].non_tensor_batch
        rm = nt.get("reward_model") or {}
        extra = dict(nt.get("extra_info") or {})
        extra["num_turns"] = nt.get("__num_turns__")
        extra["rollout_reward_scores"] = nt.get("reward_scores", {})
        res = await self._score(data_source=nt.get("data_source"), solution_str=response,
                                ground_truth=rm.get("ground_truth") if isinstance(rm, dict) else None, extra_info=extra)
        return self._pack(res)


@register("dapo")
class DAPORewardManager(NaiveRewardManager):
    """Adds the soft overlong penalty (``reward_model.overlong_buffer``: len, penalty_factor, enable)."""

    async def run_single(self, data: DataProto) -> dict:
        out = await super().run_single(data)
        ob = _rm_cfg(self.config).get("overlong_buffer") or (_rm_cfg(self.config).get("reward_kwargs") or {}).get("overlong_buffer_cfg")
        if ob and ob.get("enable", False):
            _, _, valid = self._decode(data)
            max_len = int(_rm_cfg(self.config).get("max_resp_len") or data.batch["responses"].shape[-1])
            buf = int(ob["len"])
            exceed = valid - (max_len - buf)
            penalty = min(-exceed / buf * float(ob["penalty_factor"]), 0.0)
            out["reward_score"] += penalty
            if ob.get("log", False):
                out["reward_extra_info"].update(overlong_reward=penalty, overlong=penalty < 0)
        return out


class AsyncTokenBucket:
    """Token bucket with fractional / variable consumption. Starts full, refills at ``rate_limit`` per second, capacity
    ``max_tokens``; ``acquire(n)`` sleeps until n tokens are there (a request larger than the capacity drives the
    level negative after waiting for it at the refill rate)."""

    def __init__(self, rate_limit: float, max_tokens: Optional[float] = None):
        self.rate_limit = float(rate_limit)
        self.max_tokens = float(max_tokens or rate_limit)
        self.tokens = self.max_tokens
        self.last_update: Optional[float] = None
        self.lock = asyncio.Lock()

    async def acquire(self, num_tokens: float = 1.0) -> None:
        loop = asyncio.get_running_loop()
        while True:
            async with self.lock:
                now = loop.time()
                if self.last_update is None:
                    self.last_update = now
                self.tokens = min(self.max_tokens, self.tokens + (now - self.last_update) * self.rate_limit)
                self.last_update = now
                if self.tokens >= num_tokens:
                    self.tokens -= num_tokens
                    return
                if num_tokens > self.max_tokens:
                    # can never fit: take the debt now (later callers queue behind it) and wait it out
                    wait = (num_tokens - max(self.tokens, 0.0)) / self.rate_limit
                    self.tokens -= num_tokens
                    oversized = True
                else:
                    wait = (num_tokens - self.tokens) / self.rate_limit
                    oversized = False
            await asyncio.sleep(wait)
            if oversized:
                return


@register("rate_limited")
class RateLimitedRewardManager(NaiveRewardManager):
    """Concurrency + RPM + TPM limits shared by all instances of the process (class-level state)."""

    _semaphore: Optional[asyncio.Semaphore] = None
    _max_concurrent = None
    _rpm_limiter: Optional[AsyncTokenBucket] = None
    _tpm_limiter: Optional[AsyncTokenBucket] = None
    _max_rpm = None
    _max_tpm = None
    _estimated_tokens_per_request = 2000
    _timeout = 300.0
    _class_initialized = False

    def __init__(self, config=None, tokenizer=None, compute_score=None, reward_router_address=None, reward_model_tokenizer=None):
        super().__init__(config or {}, tokenizer, compute_score, reward_router_address, reward_model_tokenizer)
        self.init_class(config or {})

    @classmethod
    def init_class(cls, config) -> None:
        rm = _rm_cfg(config)
        if cls._class_initialized:
            if rm.get("max_rpm") != cls._max_rpm or rm.get("max_tpm") != cls._max_tpm:
                logger.warning("RateLimitedRewardManager limiters are process-wide and already set (max_rpm=%s, max_tpm=%s); "
                               "the new values (max_rpm=%s, max_tpm=%s) are ignored", cls._max_rpm, cls._max_tpm,
                               rm.get("max_rpm"), rm.get("max_tpm"))
            return
        cls._max_concurrent = int(rm.get("max_concurrent", 1))
        cls._semaphore = asyncio.Semaphore(cls._max_concurrent)
        cls._max_rpm, cls._max_tpm = rm.get("max_rpm"), rm.get("max_tpm")
        cls._rpm_limiter = AsyncTokenBucket(cls._max_rpm / 60.0, cls._max_rpm / 60.0) if cls._max_rpm else None
        cls._tpm_limiter = AsyncTokenBucket(cls._max_tpm / 60.0, cls._max_tpm / 60.0) if cls._max_tpm else None
        cls._estimated_tokens_per_request = int(rm.get("estimated_tokens_per_request", 2000))
        cls._timeout = float(rm.get("timeout", 300.0))
        cls._class_initialized = True

    @classmethod
    def reset_class(cls) -> None:
        cls._class_initialized = False
        cls._semaphore = cls._rpm_limiter = cls._tpm_limiter = None

    async def run_single(self, data: DataProto) -> dict:
        cls = type(self)
        if cls._rpm_limiter is not None:
            await cls._rpm_limiter.acquire(1.0)
        if cls._tpm_limiter is not None:
            await cls._tpm_limiter.acquire(cls._estimated_tokens_per_request)
        async with cls._semaphore:
            try:
                return await asyncio.wait_for(super().run_single(data), timeout=cls._timeout)
            except asyncio.TimeoutError:
                logger.warning("reward computation timed out after %.0f s", cls._timeout)
                return {"reward_score": 0.0, "reward_extra_info": {"timeout": True, "acc": 0.0}}
            except Exception as e:  # a failing judge call must not kill the training step
                logger.warning("reward computation failed: %s", e)
                return {"reward_score": 0.0, "reward_extra_info": {"error": str(e), "acc": 0.0}}


@register("remote")
class RemoteRewardManager(NaiveRewardManager):
    """Scores in a process pool (CPU-heavy verifiers) instead of the event loop's thread pool."""

    _pool = None

    async def _score(self, **kw):
        import concurrent.futures as cf

        cls = type(self)
        if cls._pool is None:
            cls._pool = cf.ProcessPoolExecutor(max_workers=int(_rm_cfg(self.config).get("num_workers", 4) or 4))
        loop = asyncio.get_running_loop()
        try:
            return await loop.run_in_executor(cls._pool, _call, self.compute_score, kw)
        except Exception:  # unpicklable scoring function: fall back to threads
            return await super()._score(**kw)


def _call(fn, kw):
    return fn(**kw)
