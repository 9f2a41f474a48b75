"""Worker-side profilers behind ``start_profile`` / ``stop_profile`` RPCs and ``@DistProfiler.annotate``.

Mechanism of verl/utils/profiler/profile.py:72-300 and nvtx_profile.py / torch_profile.py: the tool named in the
config (``nsys`` -> cudaProfilerStart/Stop + NVTX ranges, ``torch`` -> chrome trace per rank, ``torch_memory`` ->
allocator history snapshot) is started at the profile step on the selected ranks.
"""

from __future__ import annotations

import functools
import os
from contextlib import contextmanager
from typing import Callable, Optional

import torch


def _get(cfg, key, default=None):
    if cfg is None:
        return default
    v = cfg.get(key, default) if hasattr(cfg, "get") else getattr(cfg, key, default)
    return default if v is None else v


@contextmanager
def nvtx_range(msg: str, color: Optional[str] = None):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(msg)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


def mark_start_range(message: Optional[str] = None, **kwargs):
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(message or "range")
    return message


def mark_end_range(range_id=None):
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_pop()


def mark_annotate(message: Optional[str] = None, color: Optional[str] = None, domain: Optional[str] = None,
                  category: Optional[str] = None) -> Callable:
    """Decorator: the function runs inside an NVTX range named ``message`` (or after the function)."""

    def decorator(fn):
        @functools.wraps(fn)
        def wrapper(*args, **kw):
            with nvtx_range(message or fn.__name__, color):
                return fn(*args, **kw)

        return wrapper

    return decorator


class DistProfiler:
    """Per-rank profiler chosen by ``config.tool``; inactive ranks are no-ops."""

    def __init__(self, rank: int, config=None, tool_config=None, **kwargs):
        self.rank = rank
        self.config = config
        self.tool = _get(config, "tool", None)
        enable = bool(_get(config, "enable", False))
        ranks = _get(config, "ranks", []) or []
        self.active = enable and (bool(_get(config, "all_ranks", False)) or rank in ranks)
        self.save_path = _get(config, "save_path", "outputs/profile")
        self.tool_config = tool_config or _get(config, "tool_config", None)
        self._prof = None
        self._step = None
        self._enable, self._this_rank, self._this_step = enable, self.active, False
        # discrete mode: every annotated phase is a capture of its own instead of one capture per step
        self._discrete = bool(_get(self.tool_config, "discrete", False))

    def check_enable(self) -> bool:
        return self._enable

    def check_this_rank(self) -> bool:
        return self._this_rank

    def check_this_step(self) -> bool:
        """True between ``start`` and ``stop`` on a rank that profiles."""
        return self._this_step

    def is_discrete_mode(self) -> bool:
        return self._discrete

    def start(self, role: Optional[str] = None, profile_step: Optional[str] = None, **kwargs):
        if not self.active:
            return
        self._this_step = True
        self._step = profile_step
        if self.tool == "nsys":
            torch.cuda.profiler.start()
        elif self.tool == "torch":
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self._prof = torch.profiler.profile(activities=acts, record_shapes=True)
            self._prof.start()
            self._role = role
        elif self.tool == "torch_memory" and torch.cuda.is_available():
            torch.cuda.memory._record_memory_history(max_entries=int(_get(self.tool_config, "trace_alloc_max_entries", 100000)))

    def stop(self):
        if not self.active:
            return
        self._this_step = False
        if self.tool == "nsys":
            torch.cuda.profiler.stop()
        elif self.tool == "torch" and self._prof is not None:
            self._prof.stop()
            os.makedirs(self.save_path, exist_ok=True)
            name = f"prof_rank-{self.rank}" + (f"_step-{self._step}" if self._step is not None else "") + ".json.gz"
            self._prof.export_chrome_trace(os.path.join(self.save_path, name))
            self._prof = None
        elif self.tool == "torch_memory" and torch.cuda.is_available():
            os.makedirs(self.save_path, exist_ok=True)
            torch.cuda.memory._dump_snapshot(os.path.join(self.save_path, f"memory_rank-{self.rank}.pickle"))
            torch.cuda.memory._record_memory_history(enabled=None)

    @classmethod
    def annotate(cls, message: Optional[str] = None, color: Optional[str] = None, role: Optional[str] = None,
                 **kwargs) -> Callable:
        """Decorator that wraps a worker method in an NVTX range named after it."""

        def deco(fn):
            @functools.wraps(fn)
            def wrapper(self, *args, **kw):
                with nvtx_range(message or fn.__name__, color):
                    return fn(self, *args, **kw)

            return wrapper

        return deco


class DistProfilerExtension:
    """Mixin giving a worker ``start_profile`` / ``stop_profile`` (ONE_TO_ALL RPCs in the reference)."""

    def __init__(self, profiler: DistProfiler):
        self.profiler = profiler

    def start_profile(self, **kwargs):
        self.profiler.start(**kwargs)

    def stop_profile(self):
        self.profiler.stop()
