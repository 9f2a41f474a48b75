"""A small batch-of-tensors container with the subset of ``tensordict.TensorDict``
semantics the framework relies on (the reference depends on the external
``tensordict`` package: verl/protocol.py, verl/utils/tensordict_utils.py).

A :class:`TensorDict` maps names to tensors that share their leading ``batch_size``
dimensions. Entries may also be jagged ``torch.nested`` tensors (leading dim only) or
:class:`NonTensorData` / :class:`NonTensorStack` for Python payloads that must travel
with the batch. Indexing, chunk/split/cat, device moves and key selection apply to
every entry at once.
"""

from __future__ import annotations

from typing import Any, Iterable, Iterator, Sequence

import numpy as np
import torch


class NonTensorData:
    """A Python object shared by the whole batch (not indexed)."""

    __slots__ = ("data",)

    def __init__(self, data: Any):
        self.data = data

    def __repr__(self):
        return f"NonTensorData({self.data!r})"

    def __eq__(self, other):
        return isinstance(other, NonTensorData) and self.data == other.data


class NonTensorStack:
    """One Python object per batch element (indexed with the batch)."""

    __slots__ = ("items",)

    def __init__(self, items: Sequence[Any]):
        self.items = list(items)

    def __len__(self):
        return len(self.items)

    def tolist(self):
        return list(self.items)

    def __repr__(self):
        return f"NonTensorStack(n={len(self.items)})"

    def _index(self, idx):
        if isinstance(idx, (int, np.integer)):
            return self.items[int(idx)]
        if isinstance(idx, slice):
            return NonTensorStack(self.items[idx])
        if isinstance(idx, torch.Tensor):
            if idx.dtype == torch.bool:
                idx = torch.nonzero(idx, as_tuple=False).flatten()
            idx = idx.tolist()
        if isinstance(idx, np.ndarray):
            if idx.dtype == bool:
                idx = np.nonzero(idx)[0]
            idx = idx.tolist()
        return NonTensorStack([self.items[i] for i in idx])


def _is_nested(t) -> bool:
    return isinstance(t, torch.Tensor) and t.is_nested


def _index_value(v, idx):
    if isinstance(v, NonTensorData):
        return v
    if isinstance(v, NonTensorStack):
        return v._index(idx)
    if _is_nested(v):
        if isinstance(idx, (int, np.integer)):
            return v[int(idx)]
        if isinstance(idx, slice):
            rows = list(v.unbind(0))[idx]
        else:
            if isinstance(idx, torch.Tensor):
                if idx.dtype == torch.bool:
                    idx = torch.nonzero(idx, as_tuple=False).flatten()
                idx = idx.tolist()
            elif isinstance(idx, np.ndarray):
                if idx.dtype == bool:
                    idx = np.nonzero(idx)[0]
                idx = idx.tolist()
            rows_all = list(v.unbind(0))
            rows = [rows_all[i] for i in idx]
        return torch.nested.as_nested_tensor(rows, layout=torch.jagged) if rows else rows
    if isinstance(idx, np.ndarray):
        idx = torch.from_numpy(idx)
    if isinstance(idx, list):
        idx = torch.as_tensor(idx)
    if isinstance(idx, torch.Tensor) and idx.device != v.device:
        idx = idx.to(v.device)
    return v[idx]


class TensorDict:
    def __init__(self, source: dict | None = None, batch_size: Sequence[int] | int | None = None, device=None):
        self._data: dict[str, Any] = {}
        if batch_size is None:
            batch_size = ()
        if isinstance(batch_size, int):
            batch_size = (batch_size,)
        self._batch_size = torch.Size(batch_size)
        if source:
            for k, v in source.items():
                self[k] = v
        if device is not None:
            self._data = self.to(device)._data

    # ------------------------------------------------------------------ basics
    @property
    def batch_size(self) -> torch.Size:
        return self._batch_size

    @batch_size.setter
    def batch_size(self, value):
        value = torch.Size((value,) if isinstance(value, int) else value)
        for k, v in self._data.items():
            if isinstance(v, torch.Tensor) and not v.is_nested and tuple(v.shape[: len(value)]) != tuple(value):
                raise RuntimeError(f"batch_size {tuple(value)} incompatible with entry {k!r} of shape {tuple(v.shape)}")
        self._batch_size = value

    @property
    def batch_dims(self) -> int:
        return len(self._batch_size)

    @property
    def device(self):
        for v in self._data.values():
            if isinstance(v, torch.Tensor):
                return v.device
        return None

    def keys(self):
        return self._data.keys()

    def values(self):
        return self._data.values()

    def items(self):
        return self._data.items()

    def __contains__(self, key) -> bool:
        return key in self._data

    def __iter__(self) -> Iterator:
        if not self._batch_size:
            raise TypeError("iteration over a TensorDict without batch dimension")
        for i in range(self._batch_size[0]):
            yield self[i]

    def __len__(self) -> int:
        return self._batch_size[0] if self._batch_size else 0

    def numel(self) -> int:
        n = 1
        for s in self._batch_size:
            n *= s
        return n

    def is_empty(self) -> bool:
        return len(self._data) == 0

    def get(self, key, default=None):
        return self._data.get(key, default)

    def __getitem__(self, idx):
        if isinstance(idx, str):
            return self._data[idx]
        if isinstance(idx, tuple) and idx and all(isinstance(k, str) for k in idx):
            raise KeyError("nested keys are not supported")
        new = TensorDict.__new__(TensorDict)
        new._data = {k: _index_value(v, idx) for k, v in self._data.items()}
        new._batch_size = self._indexed_batch_size(idx)
        return new

    def _indexed_batch_size(self, idx) -> torch.Size:
        if not self._batch_size:
            raise IndexError("cannot index a TensorDict with empty batch_size")
        probe = torch.empty(self._batch_size, device="meta")
        if isinstance(idx, np.ndarray):
            idx = torch.from_numpy(idx)
        if isinstance(idx, torch.Tensor):
            idx = idx.to("cpu")
            if idx.dtype == torch.bool:
                return torch.Size((int(idx.sum()),) + tuple(self._batch_size[idx.dim():]))
            return torch.Size(tuple(idx.shape) + tuple(self._batch_size[1:]))
        if isinstance(idx, list):
            return torch.Size((len(idx),) + tuple(self._batch_size[1:]))
        return probe[idx].shape

    def __setitem__(self, key: str, value):
        if not isinstance(key, str):
            raise KeyError("only string keys can be assigned")
        if isinstance(value, np.ndarray) and value.dtype != object:
            value = torch.from_numpy(value)
        if isinstance(value, torch.Tensor):
            nb = len(self._batch_size)
            if value.is_nested:
                if nb and value.size(0) != self._batch_size[0]:
                    raise RuntimeError(f"nested entry {key!r} has {value.size(0)} rows, batch is {self._batch_size[0]}")
            elif tuple(value.shape[:nb]) != tuple(self._batch_size):
                raise RuntimeError(
                    f"entry {key!r} with shape {tuple(value.shape)} does not start with batch_size {tuple(self._batch_size)}"
                )
            self._data[key] = value
        elif isinstance(value, (NonTensorData, NonTensorStack)):
            if isinstance(value, NonTensorStack) and self._batch_size and len(value) != self._batch_size[0]:
                raise RuntimeError(f"NonTensorStack {key!r} has {len(value)} items, batch is {self._batch_size[0]}")
            self._data[key] = value
        elif isinstance(value, (list, tuple)) and self._batch_size and len(value) == self._batch_size[0]:
            self._data[key] = NonTensorStack(value)
        elif isinstance(value, np.ndarray):
            self._data[key] = NonTensorStack(list(value))
        else:
            self._data[key] = NonTensorData(value)

    def set(self, key, value):
        self[key] = value
        return self

    def pop(self, key, *default):
        return self._data.pop(key, *default)

    def __delitem__(self, key):
        del self._data[key]

    def update(self, other: "TensorDict | dict"):
        for k, v in other.items():
            self[k] = v
        return self

    def rename_key_(self, old: str, new: str):
        self._data[new] = self._data.pop(old)
        return self

    # ------------------------------------------------------------- projections
    def select(self, *keys: str, strict: bool = True) -> "TensorDict":
        new = TensorDict.__new__(TensorDict)
        new._batch_size = self._batch_size
        if strict:
            missing = [k for k in keys if k not in self._data]
            if missing:
                raise KeyError(f"keys {missing} not found")
        new._data = {k: self._data[k] for k in keys if k in self._data}
        return new

    def exclude(self, *keys: str) -> "TensorDict":
        new = TensorDict.__new__(TensorDict)
        new._batch_size = self._batch_size
        new._data = {k: v for k, v in self._data.items() if k not in keys}
        return new

    def _map(self, fn) -> "TensorDict":
        new = TensorDict.__new__(TensorDict)
        new._batch_size = self._batch_size
        new._data = {k: (fn(v) if isinstance(v, torch.Tensor) else v) for k, v in self._data.items()}
        return new

    def to(self, device, non_blocking: bool = False) -> "TensorDict":
        return self._map(lambda t: t.to(device, non_blocking=non_blocking))

    def cpu(self):
        return self.to("cpu")

    def cuda(self, device=None):
        return self.to("cuda" if device is None else device)

    def clone(self) -> "TensorDict":
        return self._map(lambda t: t.clone())

    def contiguous(self) -> "TensorDict":
        return self._map(lambda t: t if t.is_nested else t.contiguous())

    def consolidate(self) -> "TensorDict":
        return self.contiguous()

    def detach(self):
        return self._map(lambda t: t.detach())

    def pin_memory(self):
        return self._map(lambda t: t if t.is_nested else t.pin_memory())

    def view(self, *shape):
        shape = shape[0] if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)) else shape
        nb = len(self._batch_size)
        new = TensorDict.__new__(TensorDict)
        new._data = {
            k: (v.reshape(*shape, *v.shape[nb:]) if isinstance(v, torch.Tensor) else v) for k, v in self._data.items()
        }
        new._batch_size = torch.empty(self._batch_size, device="meta").reshape(*shape).shape
        return new

    reshape = view

    # ---------------------------------------------------------------- splitting
    def split(self, split_size: int | Sequence[int], dim: int = 0) -> list["TensorDict"]:
        if dim != 0:
            raise NotImplementedError("split along dim 0 only")
        n = self._batch_size[0]
        sizes = [min(split_size, n - s) for s in range(0, n, split_size)] if isinstance(split_size, int) else list(split_size)
        out, start = [], 0
        for s in sizes:
            out.append(self[start : start + s])
            start += s
        return out

    def chunk(self, chunks: int, dim: int = 0) -> list["TensorDict"]:
        n = self._batch_size[0]
        size = (n + chunks - 1) // chunks if n else 1
        return self.split(size, dim)

    def unbind(self, dim: int = 0) -> list["TensorDict"]:
        return [self[i] for i in range(self._batch_size[0])]

    def repeat_interleave(self, repeats: int, dim: int = 0) -> "TensorDict":
        idx = torch.arange(self._batch_size[0]).repeat_interleave(repeats)
        return self[idx]

    # ---------------------------------------------------------------- combining
    @staticmethod
    def cat(tds: Sequence["TensorDict"], dim: int = 0) -> "TensorDict":
        if dim != 0:
            raise NotImplementedError("cat along dim 0 only")
        tds = [t for t in tds if t is not None]
        if not tds:
            raise ValueError("nothing to concatenate")
        keys = list(tds[0].keys())
        new = TensorDict.__new__(TensorDict)
        new._data = {}
        for k in keys:
            vals = [t._data[k] for t in tds]
            v0 = vals[0]
            if isinstance(v0, NonTensorData):
                new._data[k] = v0
            elif isinstance(v0, NonTensorStack):
                new._data[k] = NonTensorStack([x for v in vals for x in v.items])
            elif _is_nested(v0):
                rows = [r for v in vals for r in v.unbind(0)]
                new._data[k] = torch.nested.as_nested_tensor(rows, layout=torch.jagged)
            else:
                new._data[k] = torch.cat(vals, dim=0)
        if len(tds[0]._batch_size) == 0:  # no batch dimension (results that carry only batch-level data)
            new._batch_size = torch.Size(())
            return new
        total = sum(t._batch_size[0] for t in tds)
        new._batch_size = torch.Size((total,) + tuple(tds[0]._batch_size[1:]))
        return new

    @staticmethod
    def stack(tds: Sequence["TensorDict"], dim: int = 0) -> "TensorDict":
        keys = list(tds[0].keys())
        new = TensorDict.__new__(TensorDict)
        new._data = {}
        for k in keys:
            vals = [t._data[k] for t in tds]
            if isinstance(vals[0], torch.Tensor):
                new._data[k] = torch.stack(vals, dim=dim)
            elif isinstance(vals[0], NonTensorData):
                new._data[k] = NonTensorStack([v.data for v in vals])
            else:
                new._data[k] = NonTensorStack(vals)
        new._batch_size = torch.Size((len(tds),) + tuple(tds[0]._batch_size))
        return new

    def to_dict(self) -> dict:
        return dict(self._data)

    def __repr__(self):
        body = ", ".join(
            f"{k}: {tuple(v.shape) if isinstance(v, torch.Tensor) and not v.is_nested else type(v).__name__}"
            for k, v in self._data.items()
        )
        return f"TensorDict({{{body}}}, batch_size={tuple(self._batch_size)})"

    # pickling keeps plain tensors (moved through torch's own reducer)
    def __getstate__(self):
        return {"data": self._data, "batch_size": tuple(self._batch_size)}

    def __setstate__(self, state):
        self._data = state["data"]
        self._batch_size = torch.Size(state["batch_size"])


def is_tensordict(obj) -> bool:
    return isinstance(obj, TensorDict)


def cat(tds: Iterable[TensorDict], dim: int = 0) -> TensorDict:
    return TensorDict.cat(list(tds), dim)
