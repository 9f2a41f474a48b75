"""Kept for import compatibility (verl/utils/debug/performance.py re-exports the profiler helpers)."""

from ..profiler.performance import GPUMemoryLogger, log_gpu_memory_usage, log_print  # noqa: F401
