"""Trainer-side adapter to the native rollout engine (role of ``ServerAdapter`` in
verl/workers/rollout/vllm_rollout/vllm_rollout.py:62-232).

The reference ships weights to a separate vLLM process through CUDA-IPC buckets and a ZMQ handshake. Here the
engine lives in the trainer's process on the same GPU, so ``update_weights`` writes straight into the engine's
parameters (or does nothing when they alias the trainer's tensors)."""

from __future__ import annotations

from typing import Generator, Optional

import torch

from ...rollout import NativeRolloutEngine
from .base import BaseRollout


class ServerAdapter(BaseRollout):
    def __init__(self, config, model_config, device_mesh=None, engine: Optional[NativeRolloutEngine] = None):
        super().__init__(config, model_config, device_mesh)
        self.engine = engine

    def attach(self, engine: NativeRolloutEngine):
        self.engine = engine

    async def resume(self, tags: list[str]):
        self.engine.wake_up(tags)

    async def release(self):
        self.engine.sleep()

    async def update_weights(self, weights: Generator[tuple[str, torch.Tensor], None, None], peft_config=None,
                             base_sync_done: bool = False, **kwargs):
        self.engine.update_weights(weights)

    def generate_sequences(self, prompts):
        raise NotImplementedError("batch generation goes through ActorRolloutRefWorker.generate_sequences")
