from .base import (CheckpointEngine, CheckpointEngineManager, CheckpointEngineRegistry, CheckpointEngineWithCache,
                   ColocatedCheckpointEngine, NCCLCheckpointEngine, NVLinkCheckpointEngine, TensorMeta)
from .pinned_bucket import PinnedBucketEngine, plan_buckets

__all__ = ["CheckpointEngine", "CheckpointEngineManager", "CheckpointEngineRegistry", "CheckpointEngineWithCache",
           "ColocatedCheckpointEngine", "NCCLCheckpointEngine", "NVLinkCheckpointEngine", "PinnedBucketEngine",
           "TensorMeta", "plan_buckets"]
