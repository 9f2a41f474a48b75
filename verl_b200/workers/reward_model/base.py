"""Interface of a model-based reward (verl/workers/reward_model/base.py:1-58). The worker that serves one is
``verl_b200.workers.engine_workers.RewardModelWorker``."""

from __future__ import annotations

from abc import ABC, abstractmethod

from ...protocol import DataProto

__all__ = ["BasePPORewardModel"]


class BasePPORewardModel(ABC):
    def __init__(self, config):
        self.config = config

    @abstractmethod
    def compute_reward(self, data: DataProto) -> DataProto:
        """``data.batch``: ``input_ids``, ``attention_mask``, ``position_ids`` of prompt + response. Returns a DataProto
        whose batch has ``rm_scores`` ``[batch, response_length]`` (the score on the last valid response token for a
        sequence-level model)."""
