"""Column store data plane between the controller and the workers.

Role of verl/experimental/transfer_queue/ and verl/utils/transferqueue_utils.py (``@tqbridge``): instead of shipping
whole ``DataProto`` batches through the controller, the trainer passes a small ``BatchMeta`` (row ids + column names);
a worker method decorated with ``@tqbridge`` fetches exactly the columns it reads, runs, and writes the columns it
produced back, returning a new ``BatchMeta``. The reference talks to the external TransferQueue service; this is
the same contract on an in-process (thread-safe) store, which is what a single-node run needs. Rows are addressed by
a global index; every column remembers which rows are filled, so consumers can wait for producers
(``get(..., timeout)``) — the streaming behaviour the asynchronous trainers build on.
"""

from __future__ import annotations

import functools
import inspect
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Optional

import numpy as np
import torch

from ...protocol import DataProto


@dataclass
class BatchMeta:
    global_indexes: list[int]
    columns: list[str] = field(default_factory=list)
    meta_info: dict = field(default_factory=dict)

    def __len__(self) -> int:
        return len(self.global_indexes)

    def select(self, columns: list[str]) -> "BatchMeta":
        return BatchMeta(list(self.global_indexes), [c for c in columns if c in self.columns], dict(self.meta_info))

    def chunk(self, n: int) -> list["BatchMeta"]:
        assert len(self) % n == 0, "only equal chunks"
        k = len(self) // n
        return [BatchMeta(self.global_indexes[i * k : (i + 1) * k], list(self.columns), dict(self.meta_info)) for i in range(n)]

    @staticmethod
    def concat(parts: list["BatchMeta"]) -> "BatchMeta":
        cols: list[str] = []
        for p in parts:
            cols += [c for c in p.columns if c not in cols]
        info: dict = {}
        for p in parts:
            info.update(p.meta_info)
        return BatchMeta([i for p in parts for i in p.global_indexes], cols, info)

    def union(self, other: "BatchMeta") -> "BatchMeta":
        assert self.global_indexes == other.global_indexes
        return BatchMeta(list(self.global_indexes), self.columns + [c for c in other.columns if c not in self.columns],
                         {**self.meta_info, **other.meta_info})


class TransferQueue:
    def __init__(self):
        self._tensors: dict[str, dict[int, torch.Tensor]] = {}
        self._objects: dict[str, dict[int, Any]] = {}
        self._cv = threading.Condition()
        self._next = 0
        self.bytes_put = self.bytes_get = 0

    def allocate(self, n: int) -> list[int]:
        with self._cv:
            ids = list(range(self._next, self._next + n))
            self._next += n
            return ids

    def put(self, indexes: list[int], data: DataProto) -> list[str]:
        assert len(indexes) == len(data)
        cols = []
        with self._cv:
            if data.batch is not None:
                for k in data.batch.keys():
                    col = self._tensors.setdefault(k, {})
                    t = data.batch[k]
                    for j, i in enumerate(indexes):
                        col[i] = t[j].clone()
                    self.bytes_put += t.numel() * t.element_size()
                    cols.append(k)
            for k, v in data.non_tensor_batch.items():
                col = self._objects.setdefault(k, {})
                for j, i in enumerate(indexes):
                    col[i] = v[j]
                cols.append(k)
            self._cv.notify_all()
        return cols

    def _ready(self, indexes, columns) -> bool:
        for c in columns:
            col = self._tensors.get(c) if c in self._tensors else self._objects.get(c)
            if col is None or any(i not in col for i in indexes):
                return False
        return True

    def get(self, indexes: list[int], columns: list[str], timeout: Optional[float] = None) -> DataProto:
        deadline = None if timeout is None else time.monotonic() + timeout
        with self._cv:
            while not self._ready(indexes, columns):
                left = None if deadline is None else deadline - time.monotonic()
                if left is not None and left <= 0:
                    raise TimeoutError(f"columns {columns} are not complete for the requested rows")
                self._cv.wait(left)
            tensors, objects = {}, {}
            for c in columns:
                if c in self._tensors:
                    tensors[c] = torch.stack([self._tensors[c][i] for i in indexes])
                    self.bytes_get += tensors[c].numel() * tensors[c].element_size()
                else:
                    arr = np.empty(len(indexes), dtype=object)
                    arr[:] = [self._objects[c][i] for i in indexes]
                    objects[c] = arr
        return DataProto.from_dict(tensors=tensors or None, non_tensors=objects or None)

    def clear(self, indexes: Optional[list[int]] = None) -> None:
        with self._cv:
            for col in list(self._tensors.values()) + list(self._objects.values()):
                if indexes is None:
                    col.clear()
                else:
                    for i in indexes:
                        col.pop(i, None)


_QUEUE: Optional[TransferQueue] = None


def set_transfer_queue(q: Optional[TransferQueue]) -> None:
    global _QUEUE
    _QUEUE = q


def get_transfer_queue() -> TransferQueue:
    global _QUEUE
    if _QUEUE is None:
        _QUEUE = TransferQueue()
    return _QUEUE


def tqbridge(reads: Optional[list[str]] = None, writes_meta: bool = True):
    """Worker-method decorator: ``BatchMeta`` arguments become ``DataProto`` (only the columns in ``reads``, or all the
    columns the meta lists), a returned ``DataProto`` is stored and replaced by a ``BatchMeta`` of the same rows.
    Calls that pass ``DataProto`` directly are left alone, so a method works in both data planes."""

    def deco(fn):
        def convert_in(v):
            if isinstance(v, BatchMeta):
                cols = [c for c in (reads or v.columns) if c in v.columns]
                d = get_transfer_queue().get(v.global_indexes, cols)
                d.meta_info = dict(v.meta_info)
                return d, v
            return v, None

        def convert_out(out, meta: Optional[BatchMeta]):
            if meta is None or not isinstance(out, DataProto) or not writes_meta:
                return out
            cols = get_transfer_queue().put(meta.global_indexes, out) if len(out) == len(meta) else []
            return BatchMeta(list(meta.global_indexes), cols, dict(out.meta_info))

        if inspect.iscoroutinefunction(fn):
            @functools.wraps(fn)
            async def awrapper(self, *args, **kwargs):
                metas = []
                args = list(args)
                for i, a in enumerate(args):
                    args[i], m = convert_in(a)
                    metas.append(m)
                for k in list(kwargs):
                    kwargs[k], m = convert_in(kwargs[k])
                    metas.append(m)
                return convert_out(await fn(self, *args, **kwargs), next((m for m in metas if m is not None), None))

            return awrapper

        @functools.wraps(fn)
        def wrapper(self, *args, **kwargs):
            metas = []
            args = list(args)
            for i, a in enumerate(args):
                args[i], m = convert_in(a)
                metas.append(m)
            for k in list(kwargs):
                kwargs[k], m = convert_in(kwargs[k])
                metas.append(m)
            return convert_out(fn(self, *args, **kwargs), next((m for m in metas if m is not None), None))

        return wrapper

    return deco
