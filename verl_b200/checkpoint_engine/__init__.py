from .base import (CheckpointEngine, CheckpointEngineManager, CheckpointEngineRegistry, CheckpointEngineWithCache,
                   CheckpointEngineWorker,
                   ColocatedCheckpointEngine, NCCLCheckpointEngine, NVLinkCheckpointEngine, TensorMeta,
                   build_checkpoint_engine)
from .pinned_bucket import PinnedBucketEngine, plan_buckets

__all__ = ["CheckpointEngine", "CheckpointEngineManager", "CheckpointEngineWorker", "CheckpointEngineRegistry", "CheckpointEngineWithCache",
           "ColocatedCheckpointEngine", "NCCLCheckpointEngine", "NVLinkCheckpointEngine", "PinnedBucketEngine",
           "TensorMeta", "build_checkpoint_engine", "plan_buckets"]
