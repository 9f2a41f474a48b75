"""Custom / curriculum sampler interfaces (verl/experimental/dataset/sampler.py:23-40), plus one concrete curriculum
sampler that the reference leaves to the user: it re-weights prompts by how informative their last rollouts were.

A sampler named in ``data.sampler.class_path`` / ``class_name`` is built by the trainer entry point with
``(data_source, data_config)``; when it is a curriculum sampler the trainer calls ``update(batch)`` after every step
(``data.dataloader_num_workers`` must then be 0 so that the sampler object the trainer updates is the one that samples).
"""

from __future__ import annotations

from abc import abstractmethod
from typing import Iterator, Sized

import numpy as np
from torch.utils.data import Sampler


class AbstractSampler(Sampler[int]):
    @abstractmethod
    def __init__(self, data_source: Sized, data_config):
        pass


class AbstractCurriculumSampler(AbstractSampler):
    @abstractmethod
    def update(self, batch) -> None:
        """Called with the finished training batch (a ``DataProto``) after each step."""


class DifficultyCurriculumSampler(AbstractCurriculumSampler):
    """Samples prompts with probability proportional to ``p (1 - p) + floor`` where ``p`` is the running mean
    sequence score of the prompt: prompts that are always solved or never solved give no GRPO signal and fade out."""

    def __init__(self, data_source: Sized, data_config):
        self.n = len(data_source)
        sc = (data_config.get("sampler") or {}) if hasattr(data_config, "get") else {}
        self.floor = float(sc.get("floor", 0.05))
        self.momentum = float(sc.get("momentum", 0.5))
        self.chunk = max(1, int(sc.get("refresh_every", 256)))
        self.rng = np.random.default_rng(int(data_config.get("seed", 1) or 1) if hasattr(data_config, "get") else 1)
        self.p = np.full(self.n, 0.5)

    def __len__(self) -> int:
        return self.n

    def __iter__(self) -> Iterator[int]:
        left = self.n
        while left > 0:  # weights are refreshed every ``chunk`` draws (one O(n) pass per chunk, not per sample)
            k = min(left, self.chunk)
            w = self.p * (1 - self.p) + self.floor
            for i in self.rng.choice(self.n, size=k, p=w / w.sum()):
                yield int(i)
            left -= k

    def update(self, batch) -> None:
        idx = batch.non_tensor_batch.get("index")
        if idx is None or "token_level_scores" not in batch.batch.keys():
            return
        score = batch.batch["token_level_scores"].sum(-1).float().cpu().numpy()
        for i, s in zip(idx, score):
            i = int(i) % self.n
            self.p[i] = self.momentum * self.p[i] + (1 - self.momentum) * float(np.clip(s, 0.0, 1.0))
