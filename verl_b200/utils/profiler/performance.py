"""Memory logging and stage timers (verl/utils/profiler/performance.py:29-260)."""

from __future__ import annotations

import datetime
import inspect
import logging
import time
from contextlib import contextmanager
from typing import Any, Optional

import torch
import torch.distributed as dist

from ..logger.aggregate_logger import DecoratorLoggerBase
from .profile import nvtx_range


def _get_current_mem_info(unit: str = "GB", precision: int = 2) -> tuple[str, str, str, str]:
    div = {"GB": 1024**3, "MB": 1024**2, "KB": 1024}[unit]
    if not torch.cuda.is_available():
        return ("0",) * 4
    free, total = torch.cuda.mem_get_info()
    f = lambda v: f"{v / div:.{precision}f}"  # noqa: E731
    return f(torch.cuda.memory_allocated()), f(torch.cuda.memory_reserved()), f(total - free), f(total)


def log_gpu_memory_usage(head: str, logger: Optional[logging.Logger] = None, level=logging.DEBUG, rank: int = 0):
    if dist.is_initialized() and rank is not None and dist.get_rank() != rank:
        return
    alloc, reserved, used, total = _get_current_mem_info()
    msg = f"{head}, memory allocated (GB): {alloc}, memory reserved (GB): {reserved}, device memory used/total (GB): {used}/{total}"
    if logger is None:
        print(msg, flush=True)
    else:
        logger.log(level, msg)


class GPUMemoryLogger(DecoratorLoggerBase):
    """``@GPUMemoryLogger(role="actor")`` logs device memory before and after the decorated call."""

    def __init__(self, role: str, logger: Optional[logging.Logger] = None, level=logging.DEBUG, log_only_rank_0: bool = True):
        super().__init__(role, logger, level, None, log_only_rank_0)

    def __call__(self, fn):
        if inspect.iscoroutinefunction(fn):
            async def wrapped(*a, **k):
                self._log(fn.__name__, "Before")
                out = await fn(*a, **k)
                self._log(fn.__name__, "After")
                return out
        else:
            def wrapped(*a, **k):
                self._log(fn.__name__, "Before")
                out = fn(*a, **k)
                self._log(fn.__name__, "After")
                return out
        wrapped.__name__, wrapped.__doc__ = fn.__name__, fn.__doc__
        return wrapped

    def _log(self, name: str, when: str):
        alloc, reserved, used, total = _get_current_mem_info()
        self.logging_function(f"{when} {name}, memory allocated (GB): {alloc}, memory reserved (GB): {reserved}, "
                              f"device memory used/total (GB): {used}/{total}")


def log_print(ctn: Any):
    frame = inspect.currentframe().f_back
    print(f"[{datetime.datetime.now():%Y-%m-%d %H:%M:%S}-{frame.f_code.co_filename.split('/')[-1]}:{frame.f_lineno}"
          f":{frame.f_code.co_name}]: {ctn}")


@contextmanager
def simple_timer(name: str, timing_raw: dict[str, float]):
    t0 = time.perf_counter()
    yield
    timing_raw[name] = timing_raw.get(name, 0.0) + time.perf_counter() - t0


@contextmanager
def marked_timer(name: str, timing_raw: dict[str, float], color: Optional[str] = None, **kwargs):
    with nvtx_range(name, color), simple_timer(name, timing_raw):
        yield


def _device():
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and dist.get_backend() == "nccl" else torch.device("cpu")


def reduce_timing(timing_raw: dict[str, float], reduce_op=None) -> dict[str, float]:
    """Average (default) every timer over the ranks."""
    if not dist.is_initialized():
        return timing_raw
    keys = sorted(timing_raw)
    t = torch.tensor([timing_raw[k] for k in keys], dtype=torch.float32, device=_device())
    avg = reduce_op is None or reduce_op == dist.ReduceOp.AVG
    dist.all_reduce(t, op=dist.ReduceOp.SUM if avg else reduce_op)  # gloo has no AVG
    if avg:
        t /= dist.get_world_size()
    return dict(zip(keys, t.cpu().tolist()))


def topk_reduce_ratio_min_max(timing: float, k: int = 10) -> tuple[float, float, float]:
    """(share of ranks slower than the (100-k)-th percentile, min, max) of one timer over the ranks."""
    if not dist.is_initialized():
        return -1.0, -1.0, -1.0
    mine = torch.tensor([timing], dtype=torch.float32, device=_device())
    parts = [torch.zeros_like(mine) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, mine)
    s = torch.cat(parts).cpu()
    top = torch.quantile(s, 1 - k / 100)
    return (s > top).float().mean().item(), s.min().item(), s.max().item()


def gather_timing(timing_raw: dict[str, float]) -> dict[str, list[float]]:
    if not dist.is_initialized():
        return {k: [v] for k, v in timing_raw.items()}
    keys = sorted(timing_raw)
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, [timing_raw[k] for k in keys])
    return {k: [r[i] for r in out] for i, k in enumerate(keys)}
