"""Parameter synchroniser of the fully asynchronous pipeline: pause -> sync -> resume.

Role of verl/experimental/fully_async_policy/param_sync.py:27 (``ParameterSynchronizer``): after a trainer update
the rollouter is paused (running generations are aborted and kept as partial rollouts, or drained), the new weights
are pushed to the rollout engine, the parameter version is bumped everywhere and the rollouter resumes.
"""

from __future__ import annotations

import threading
import time
from typing import Callable, Optional


class ParameterSynchronizer:
    def __init__(self, sync_fn: Callable[[int], Optional[dict]], message_queue, rollouter=None):
        self.sync_fn = sync_fn  # pushes the trainer's weights into the rollout engine, returns timing info
        self.mq = message_queue
        self.rollouter = rollouter
        self.current_version = 0
        self._lock = threading.Lock()
        self.last_sync_s = 0.0

    def get_current_param_version(self) -> int:
        return self.current_version

    def sync_weights(self, version: int, validate: bool = False) -> dict:
        with self._lock:
            t0 = time.perf_counter()
            if self.rollouter is not None:
                self.rollouter.pause()
            t1 = time.perf_counter()
            info = self.sync_fn(version) or {}
            self.current_version = int(version)
            self.mq.update_param_version(self.current_version)
            if self.rollouter is not None:
                self.rollouter.update_param_version(self.current_version)
                self.rollouter.resume()
            t2 = time.perf_counter()
            self.last_sync_s = t2 - t0
            return {"timing_s/param_sync": t2 - t0, "timing_s/param_sync_pause": t1 - t0, **{f"param_sync/{k}": v for k, v in info.items()}}


def bucket_sync_fn(engine, get_weights: Callable[[], dict], load_weights: Callable[[list], None]):
    """``sync_fn`` for :class:`ParameterSynchronizer` over a :class:`~verl_b200.checkpoint_engine.PinnedBucketEngine`:
    the trainer's current weights are staged into the pinned host buckets and streamed to ``load_weights`` (the
    rollout engine's ``update_weights``) bucket by bucket, the transfer of the next bucket overlapping the load of the
    current one (verl/experimental/fully_async_policy/checkpoint_engine.py:410, ``overlap_broadcast_and_consume``).
    A trainer that stages right after its optimizer step (``engine.stage(weights, version)``) can pass
    ``get_weights=None``: the sync then publishes what was staged."""

    def sync(version: int) -> dict:
        t0 = time.perf_counter()
        if get_weights is not None:
            w = get_weights()
            if not engine.buckets:
                engine.register([(n, tuple(t.shape), t.dtype) for n, t in w.items()])
            engine.stage(w, version=version)
        t1 = time.perf_counter()
        nbytes = engine.publish(load_weights)
        engine.version = int(version)
        return {"stage_s": t1 - t0, "publish_s": time.perf_counter() - t1, "bytes": nbytes, "buckets": len(engine.buckets)}

    return sync
