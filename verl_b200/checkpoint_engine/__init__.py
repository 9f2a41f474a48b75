from .base import (CheckpointEngine, CheckpointEngineManager, CheckpointEngineRegistry, CheckpointEngineWithCache,
                   ColocatedCheckpointEngine, NCCLCheckpointEngine, NVLinkCheckpointEngine, TensorMeta)

__all__ = ["CheckpointEngine", "CheckpointEngineManager", "CheckpointEngineRegistry", "CheckpointEngineWithCache",
           "ColocatedCheckpointEngine", "NCCLCheckpointEngine", "NVLinkCheckpointEngine", "TensorMeta"]
