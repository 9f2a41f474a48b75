from .engine import NativeRolloutEngine, SamplingParams, Scheduler, TokenOutput

__all__ = ["NativeRolloutEngine", "SamplingParams", "TokenOutput", "Scheduler"]
