"""Sample queue between the rollouter and the trainer of the fully asynchronous pipeline.

Role of verl/experimental/fully_async_policy/message_queue.py:27 (``MessageQueue`` ray actor): a bounded FIFO of
rollout samples tagged with the parameter version that produced them. ``put`` drops the oldest sample when the
queue is full, ``get`` blocks until ``n`` samples are there, samples staler than ``max_staleness`` versions are
discarded on the way out, and the counters feed the trainer's metrics.
"""

from __future__ import annotations

import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass
class QueueSample:
    data: Any
    param_version: int
    created: float = field(default_factory=time.monotonic)


class MessageQueue:
    def __init__(self, max_queue_size: int = 1024, max_staleness: Optional[int] = None):
        self.max_queue_size = int(max_queue_size)
        self.max_staleness = max_staleness
        self._q: deque[QueueSample] = deque()
        self._cv = threading.Condition()
        self.current_param_version = 0
        self.total_produced = self.total_consumed = self.dropped_full = self.dropped_stale = 0
        self._closed = False

    def put_sample(self, data: Any, param_version: int) -> bool:
        with self._cv:
            if self._closed:
                return False
            if len(self._q) >= self.max_queue_size:
                self._q.popleft()
                self.dropped_full += 1
            self._q.append(QueueSample(data, int(param_version)))
            self.total_produced += 1
            self._cv.notify_all()
            return True

    def _drop_stale(self):
        if self.max_staleness is None:
            return
        while self._q and self.current_param_version - self._q[0].param_version > self.max_staleness:
            self._q.popleft()
            self.dropped_stale += 1

    def get_samples(self, n: int, timeout: Optional[float] = None) -> Optional[list[QueueSample]]:
        """Blocks until ``n`` fresh-enough samples are available; None after ``close()`` or on timeout."""
        deadline = None if timeout is None else time.monotonic() + timeout
        with self._cv:
            while True:
                self._drop_stale()
                if len(self._q) >= n:
                    out = [self._q.popleft() for _ in range(n)]
                    self.total_consumed += n
                    self._cv.notify_all()
                    return out
                if self._closed:
                    return None
                left = None if deadline is None else deadline - time.monotonic()
                if left is not None and left <= 0:
                    return None
                self._cv.wait(left)

    def update_param_version(self, version: int) -> None:
        with self._cv:
            self.current_param_version = int(version)
            self._drop_stale()
            self._cv.notify_all()

    def get_queue_size(self) -> int:
        with self._cv:
            return len(self._q)

    def wait_below(self, size: int, timeout: Optional[float] = None) -> bool:
        """Back-pressure for the producer: wait until fewer than ``size`` samples are queued."""
        deadline = None if timeout is None else time.monotonic() + timeout
        with self._cv:
            while len(self._q) >= size and not self._closed:
                left = None if deadline is None else deadline - time.monotonic()
                if left is not None and left <= 0:
                    return False
                self._cv.wait(left)
            return not self._closed

    def get_statistics(self) -> dict:
        with self._cv:
            return {"queue_size": len(self._q), "total_produced": self.total_produced, "total_consumed": self.total_consumed,
                    "dropped_samples": self.dropped_full, "dropped_stale": self.dropped_stale,
                    "current_param_version": self.current_param_version, "max_queue_size": self.max_queue_size}

    def clear_queue(self) -> None:
        with self._cv:
            self._q.clear()
            self._cv.notify_all()

    def close(self) -> None:
        with self._cv:
            self._closed = True
            self._cv.notify_all()
