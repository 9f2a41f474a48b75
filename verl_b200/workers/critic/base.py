"""Interface of a PPO critic (verl/workers/critic/base.py): values of a batch and a value-function update."""

from __future__ import annotations

from abc import ABC, abstractmethod

import torch

from ...protocol import DataProto

__all__ = ["BasePPOCritic"]


class BasePPOCritic(ABC):
    def __init__(self, config):
        self.config = config

    @abstractmethod
    def compute_values(self, data: DataProto) -> torch.Tensor:
        """Values of the response positions ``[batch, response_length]``."""

    @abstractmethod
    def update_critic(self, data: DataProto) -> dict:
        """One update of the value function over ``data``. Returns metrics."""
