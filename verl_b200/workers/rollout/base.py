"""Rollout backend interface and registry (verl/workers/rollout/base.py:1-102).

A rollout backend lives next to a trainer worker and owns an inference engine: ``resume(tags)`` re-creates
weights / KV cache, ``update_weights(iterator of (hf_name, tensor))`` ingests new weights, ``release()`` frees
device memory, ``generate_sequences`` runs batch generation. Backends register under ``(name, mode)``.
"""

from __future__ import annotations

import importlib
from abc import ABC, abstractmethod
from typing import Generator

import torch

from ...protocol import DataProto

__all__ = ["BaseRollout", "get_rollout_class", "register_rollout"]


class BaseRollout(ABC):
    def __init__(self, config, model_config, device_mesh=None):
        self.config, self.model_config, self.device_mesh = config, model_config, device_mesh

    @abstractmethod
    async def resume(self, tags: list[str]):
        """Re-acquire device memory: ``tags`` is a subset of ["weights", "kv_cache"]."""

    @abstractmethod
    async def update_weights(self, weights: Generator[tuple[str, torch.Tensor], None, None], **kwargs):
        """Load named (HF layout) tensors into the engine."""

    @abstractmethod
    async def release(self):
        """Free weights and KV cache."""

    def generate_sequences(self, prompts: DataProto) -> DataProto:
        raise NotImplementedError


_ROLLOUT_REGISTRY: dict[tuple[str, str], str | type] = {
    ("native", "async"): "verl_b200.workers.rollout.native_rollout.ServerAdapter",
    ("native", "sync"): "verl_b200.workers.rollout.native_rollout.ServerAdapter",
    ("naive", "sync"): "verl_b200.workers.rollout.naive_rollout.NaiveRollout",
    ("hf", "sync"): "verl_b200.workers.rollout.naive_rollout.HFRollout",
    # names of the reference's engines resolve to the native engine: one code path, no backend dispatch
    ("vllm", "async"): "verl_b200.workers.rollout.native_rollout.ServerAdapter",
    ("sglang", "async"): "verl_b200.workers.rollout.native_rollout.ServerAdapter",
    ("trtllm", "async"): "verl_b200.workers.rollout.native_rollout.ServerAdapter",
}


def register_rollout(name: str, mode: str, cls):
    _ROLLOUT_REGISTRY[(name, mode)] = cls


def get_rollout_class(rollout_name: str, mode: str = "async") -> type[BaseRollout]:
    key = (rollout_name, mode)
    assert key in _ROLLOUT_REGISTRY, f"Rollout {rollout_name} with mode {mode} not found"
    target = _ROLLOUT_REGISTRY[key]
    if isinstance(target, str):
        mod, cls = target.rsplit(".", 1)
        return getattr(importlib.import_module(mod), cls)
    return target
