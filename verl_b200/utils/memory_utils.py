"""GPU memory bookkeeping helpers (role of verl/utils/memory_utils.py and debug/performance.py)."""

from __future__ import annotations

import gc

import torch


def aggressive_empty_cache(force_sync: bool = True, max_retries: int = 3) -> None:
    if not torch.cuda.is_available():
        gc.collect()
        return
    for _ in range(max_retries):
        before = torch.cuda.memory_reserved()
        gc.collect()
        torch.cuda.empty_cache()
        if force_sync:
            torch.cuda.synchronize()
        if before - torch.cuda.memory_reserved() < 64 << 20:
            break


def get_memory_info() -> dict:
    if not torch.cuda.is_available():
        return {"allocated_gb": 0.0, "reserved_gb": 0.0, "free_gb": 0.0, "total_gb": 0.0}
    free, total = torch.cuda.mem_get_info()
    return {"allocated_gb": torch.cuda.memory_allocated() / 2**30, "reserved_gb": torch.cuda.memory_reserved() / 2**30,
            "max_allocated_gb": torch.cuda.max_memory_allocated() / 2**30, "free_gb": free / 2**30, "total_gb": total / 2**30}


def log_memory_usage(stage: str = "") -> str:
    m = get_memory_info()
    line = f"[memory] {stage}: allocated {m['allocated_gb']:.2f} GB, reserved {m['reserved_gb']:.2f} GB, free {m['free_gb']:.2f} GB"
    print(line)
    return line


def enable_memory_visualize(trace_alloc_max_entries: int = 200_000, stack_depth: int = 32) -> None:
    if torch.cuda.is_available():
        torch.cuda.memory._record_memory_history(max_entries=trace_alloc_max_entries, stacks="python")


def dump_memory_snapshot(path: str) -> None:
    if torch.cuda.is_available():
        torch.cuda.memory._dump_snapshot(path)


def reset_memory_stats() -> None:
    """Reset the allocator's peak counters (before a phase whose peak is to be measured)."""
    import torch

    if torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats()
        torch.cuda.reset_accumulated_memory_stats()


class MemorySnapshotSampler:
    """Allocator snapshots of a run, one file per call, numbered, under ``out_dir/<tag>`` (viewable with
    pytorch.org/memory_viz; verl/utils/memory_utils.py ``MemorySnapshotSampler``). ``enable_memory_visualize`` must have
    switched the allocator's history on."""

    def __init__(self, out_dir: str = "./mem_snapshots", tag: str = "periodic"):
        self.out_dir, self.tag, self.count = out_dir, tag, 0

    def dump_memory_snapshot(self, out_dir: str | None = None, tag: str | None = None, sub_dir: str | None = None) -> str:
        import os

        d = os.path.join(out_dir or self.out_dir, sub_dir or "")
        os.makedirs(d, exist_ok=True)
        path = os.path.join(d, f"{tag or self.tag}_{self.count:05d}.pickle")
        self.count += 1
        dump_memory_snapshot(path)
        return path
