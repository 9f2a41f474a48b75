"""Interface of a PPO actor (verl/workers/actor/base.py): log-probs of a batch and a policy update."""

from __future__ import annotations

from abc import ABC, abstractmethod

import torch

from ...protocol import DataProto

__all__ = ["BasePPOActor"]


class BasePPOActor(ABC):
    def __init__(self, config):
        self.config = config

    @abstractmethod
    def compute_log_prob(self, data: DataProto) -> torch.Tensor:
        """``data.batch``: ``input_ids``, ``attention_mask``, ``position_ids``, ``responses``. Returns log-probs of the
        response tokens ``[batch, response_length]``."""

    @abstractmethod
    def update_policy(self, data: DataProto) -> dict:
        """One update over ``data`` (mini-batches, epochs and micro-batches as configured). Returns metrics."""
