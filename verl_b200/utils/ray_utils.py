"""Helpers the reference keeps next to its Ray glue (verl/utils/ray_utils.py:28-112). Without Ray, ``parallel_put``
hands back the objects themselves (the multi-process worker group ships arguments over its own pipes)."""

from __future__ import annotations

import asyncio
import functools
import inspect
import os
from typing import Any, Optional


def ray_noset_visible_devices(env_vars=os.environ) -> bool:
    """True if any ``RAY_EXPERIMENTAL_NOSET_*_VISIBLE_DEVICES`` variable is set."""
    return any(k.startswith("RAY_EXPERIMENTAL_NOSET_") and k.endswith("_VISIBLE_DEVICES") and v for k, v in env_vars.items())


def parallel_put(data_list: list[Any], max_workers: Optional[int] = None) -> list[Any]:
    assert len(data_list) > 0, "data_list must not be empty"
    return list(data_list)


def get_event_loop() -> asyncio.AbstractEventLoop:
    try:
        return asyncio.get_running_loop()
    except RuntimeError:
        loop = asyncio.new_event_loop()
        asyncio.set_event_loop(loop)
        return loop


def auto_await(func):
    """Call a coroutine function from sync code (runs it to completion) or from async code (returns the awaitable)."""

    @functools.wraps(func)
    def wrapper(*args, **kwargs):
        coro = func(*args, **kwargs)
        if not inspect.isawaitable(coro):
            return coro
        try:
            asyncio.get_running_loop()
        except RuntimeError:
            return asyncio.run(coro)
        return coro

    return wrapper
