"""Reward-model serving for the reward loop (role of verl/experimental/reward_loop/reward_model.py).

A discriminative reward model is a value-head engine: the score of a sample is the head's output at its last
valid token. ``RewardModelManager.score`` batches concurrent requests for a few milliseconds so that samples
scored "one at a time" by the reward loop still go through the model in packed batches.
"""

from __future__ import annotations

import asyncio
from typing import Optional

import torch

from ...models.transformer import PackedBatch
from ...protocol import DataProto


class RewardModelManager:
    def __init__(self, engine, max_batch: int = 64, max_wait_s: float = 0.005):
        self.engine = engine  # NativeEngine(value_head=True), forward only
        self.max_batch, self.max_wait_s = max_batch, max_wait_s
        self._queue: Optional[asyncio.Queue] = None
        self._task = None

    async def score(self, data: DataProto) -> float:
        if self._queue is None:
            self._queue = asyncio.Queue()
            self._task = asyncio.get_running_loop().create_task(self._serve())
        fut = asyncio.get_running_loop().create_future()
        await self._queue.put((data, fut))
        return await fut

    async def _serve(self):
        while True:
            items = [await self._queue.get()]
            t_end = asyncio.get_running_loop().time() + self.max_wait_s
            while len(items) < self.max_batch:
                left = t_end - asyncio.get_running_loop().time()
                if left <= 0:
                    break
                try:
                    items.append(await asyncio.wait_for(self._queue.get(), left))
                except asyncio.TimeoutError:
                    break
            try:
                scores = await asyncio.get_running_loop().run_in_executor(None, self._forward, [d for d, _ in items])
                for (_, fut), s in zip(items, scores):
                    fut.set_result(float(s))
            except Exception as e:
                for _, fut in items:
                    if not fut.done():
                        fut.set_exception(e)

    @torch.no_grad()
    def _forward(self, datas: list[DataProto]) -> list[float]:
        dev = self.engine.device
        ids = torch.cat([d.batch["input_ids"] for d in datas]).to(dev)
        mask = torch.cat([d.batch["attention_mask"] for d in datas]).to(dev)
        packed, _ = PackedBatch.from_padded(ids, mask)
        last_rows = packed.cu_seqlens[1:].long() - 1
        with self.engine.eval_mode():
            v = self.engine.forward_values(packed, last_rows)
        return v.float().reshape(-1).tolist()
