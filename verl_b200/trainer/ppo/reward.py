"""Reward glue: custom reward functions, reward-manager loading, synchronous / asynchronous computation
(verl/trainer/ppo/reward.py:1-216)."""

from __future__ import annotations

import inspect
import os
from concurrent.futures import ThreadPoolExecutor
from functools import partial
from typing import Any, Optional

import torch

from ...protocol import DataProto
from ...utils.py_functional import load_extern_object
from ...utils.reward_score import default_compute_score


def _call_with_kwargs(raw_fn, extra_kwargs, *args, **kwargs):
    return raw_fn(*args, **{**kwargs, **extra_kwargs})


async def _call_with_kwargs_async(raw_fn, extra_kwargs, *args, **kwargs):
    return await raw_fn(*args, **{**kwargs, **extra_kwargs})


def get_custom_reward_fn(config) -> Optional[Any]:
    """``custom_reward_function.{path,name,reward_kwargs}`` -> callable, or None when no path is set."""
    fn_cfg = config.get("custom_reward_function") or {}
    path = fn_cfg.get("path")
    if not path:
        return None
    name = fn_cfg.get("name") or "compute_score"
    raw = load_extern_object(path, name)
    kw = dict(fn_cfg.get("reward_kwargs", {}) or {})
    if inspect.iscoroutinefunction(raw):
        return partial(_call_with_kwargs_async, raw, kw)
    return partial(_call_with_kwargs, raw, kw)


def load_reward_manager(config, tokenizer, num_examine: int = 0, **reward_kwargs):
    from ...workers.reward_manager import get_reward_manager_cls

    custom = get_custom_reward_fn(config)
    rm_cfg = config.get("reward_manager") or {}
    name = rm_cfg.get("name") or (config.get("reward_model") or {}).get("reward_manager", "naive")
    if rm_cfg.get("source", "register") == "importlib":
        mod = rm_cfg.get("module") or {}
        cls = load_extern_object(mod.get("path"), mod.get("name"))
    else:
        cls = get_reward_manager_cls(name)
    score_fn = custom
    if score_fn is None:
        sf = (config.get("reward_model") or {}).get("sandbox_fusion") or {}
        if sf.get("url"):
            import threading

            sem = threading.Semaphore(int(sf.get("max_concurrent", 64)))
            score_fn = partial(default_compute_score, sandbox_fusion_url=sf["url"], concurrent_semaphore=sem,
                               memory_limit_mb=sf.get("memory_limit_mb", 1024))
        else:
            score_fn = default_compute_score
    return cls(tokenizer=tokenizer, num_examine=num_examine, compute_score=score_fn,
               reward_fn_key=config.data.get("reward_fn_key", "data_source"), **reward_kwargs)


def compute_reward(data: DataProto, reward_fn) -> tuple[torch.Tensor, dict[str, Any]]:
    try:
        res = reward_fn(data, return_dict=True)
        return res["reward_tensor"], res.get("reward_extra_info", {})
    except TypeError:
        return reward_fn(data), {}


_POOL: Optional[ThreadPoolExecutor] = None


def compute_reward_async(data: DataProto, config=None, tokenizer=None, reward_fn=None):
    """Start reward computation in the background; returns a future resolving to (reward_tensor, extra)."""
    global _POOL
    if reward_fn is None:
        assert config is not None and tokenizer is not None
        reward_fn = load_reward_manager(config, tokenizer, num_examine=0)
    if _POOL is None:
        _POOL = ThreadPoolExecutor(max_workers=2)
    return _POOL.submit(compute_reward, data, reward_fn)
