"""verl_b200: a B200-native RL post-training framework with the capabilities and public API of
volcengine/verl (single-controller WorkerGroups, DataProto, PPO/GRPO-family trainers, sharded
actor/critic/ref workers, native rollout engine, verl/HF-compatible checkpoints)."""

__version__ = "0.1.0"

from .protocol import DataProto, DataProtoFuture  # noqa: E402,F401

__all__ = ["DataProto", "DataProtoFuture", "__version__"]
