from .base import BaseRollout, get_rollout_class, register_rollout
from .replica import NativeReplica, RolloutMode, RolloutReplica, RolloutReplicaRegistry, TokenOutput, get_rollout_replica_class

__all__ = ["BaseRollout", "get_rollout_class", "register_rollout", "RolloutReplica", "RolloutMode", "NativeReplica",
           "RolloutReplicaRegistry", "get_rollout_replica_class", "TokenOutput"]
