"""Functional helpers over :class:`TensorDict` (verl/utils/tensordict_utils.py:23-870): the no-padding data path of
the reference passes ``TensorDict`` objects whose per-sample tensors are jagged nested tensors and whose Python
payloads are ``NonTensorStack`` (one per sample) or ``NonTensorData`` (one per batch)."""

from __future__ import annotations

from typing import Any, Iterable

import torch

from .tensordict_lite import NonTensorData, NonTensorStack, TensorDict


def assign_non_tensor_data(td: TensorDict, key: str, val) -> TensorDict:
    td[key] = NonTensorData(val)
    return td


def assign_non_tensor_stack(td: TensorDict, key: str, val: list) -> TensorDict:
    td[key] = NonTensorStack(list(val))
    return td


def assign_non_tensor(td: TensorDict, **kwargs) -> TensorDict:
    """Lists become per-sample stacks, everything else batch-level data."""
    for k, v in kwargs.items():
        if isinstance(v, (list, NonTensorStack)):
            assign_non_tensor_stack(td, k, v.tolist() if isinstance(v, NonTensorStack) else v)
        else:
            assign_non_tensor_data(td, k, v)
    return td


def unwrap_non_tensor_data(data):
    if isinstance(data, NonTensorData):
        return data.data
    if isinstance(data, NonTensorStack):
        return data.tolist()
    return data


def get_non_tensor_data(data: TensorDict, key: str, default):
    return unwrap_non_tensor_data(data.get(key, default))


def concat_nested_tensors(tensors: list[torch.Tensor]) -> torch.Tensor:
    rows = []
    for t in tensors:
        assert t.is_nested, "concat_nested_tensors takes nested tensors"
        rows.extend(t.unbind(0))
    return torch.nested.as_nested_tensor(rows, layout=torch.jagged)


def concat_tensordict(data: list[TensorDict]) -> TensorDict:
    assert len(data) > 0, "Must have at least one tensordict"
    return TensorDict.cat(data, 0)


def concat_tensordict_with_none_bsz(data: list[TensorDict]) -> TensorDict:
    """Results without a batch dimension (only batch-level data, e.g. per-worker metrics): the first one stands for all."""
    for d in data:
        assert len(d.batch_size) == 0, "concat_tensordict_with_none_bsz takes TensorDicts without a batch dimension"
    return data[0]


def chunk_tensordict(td: TensorDict, chunks: int) -> list[TensorDict]:
    n = td.batch_size[0]
    assert n % chunks == 0, f"expecting td with length divisible by chunks, but got {n} and {chunks}"
    return td.split(n // chunks)


def get_tensordict(tensor_dict: dict[str, torch.Tensor | list], non_tensor_dict: dict | None = None) -> TensorDict:
    bsz = None
    src = {}
    for k, v in tensor_dict.items():
        if isinstance(v, torch.Tensor) and v.is_nested:
            assert v.layout == torch.jagged, "Nested tensors must be jagged."
        if isinstance(v, list):
            assert not any(isinstance(x, torch.Tensor) for x in v), \
                "Passing a list makes the data NonTensorStack, which doesn't support torch.Tensor. Please convert to numpy first"
            v = NonTensorStack(v)
        assert isinstance(v, (torch.Tensor, NonTensorStack)), f"{k}: expected a tensor or a list, got {type(v)}"
        n = v.size(0) if isinstance(v, torch.Tensor) else len(v)
        assert bsz is None or n == bsz, f"Batch size of tensor {k} is not consistent with other tensors. Expected {bsz}, got {n}"
        bsz = n
        src[k] = v
    td = TensorDict(batch_size=[] if bsz is None else [bsz])
    for k, v in src.items():
        td[k] = v
    for k, v in (non_tensor_dict or {}).items():
        assert k not in src
        td[k] = NonTensorData(v)
    return td


def index_select_tensor_dict(batch: TensorDict, indices) -> TensorDict:
    if batch is None:
        return None
    idx = torch.as_tensor(indices)
    assert idx.dim() == 1, "indices must be a 1D tensor"
    return batch[idx]


def union_tensor_dict(td1: TensorDict, td2: TensorDict) -> TensorDict:
    assert td1.batch_size == td2.batch_size, f"Two tensor dict must have identical batch size. Got {td1.batch_size} and {td2.batch_size}"
    for k in td2.keys():
        v2 = td2.get(k)
        if k in td1:
            v1 = td1.get(k)
            if isinstance(v1, torch.Tensor) and isinstance(v2, torch.Tensor):
                same = (all(torch.equal(a, b) for a, b in zip(v1.unbind(0), v2.unbind(0))) if v1.is_nested
                        else v1.shape == v2.shape and torch.equal(v1, v2))
            else:
                same = unwrap_non_tensor_data(v1) == unwrap_non_tensor_data(v2)
            assert same, f"{k} in tensor_dict1 and tensor_dict2 are not the same object"
        else:
            td1[k] = v2
    return td1


def make_iterator(td: TensorDict, mini_batch_size: int, epochs: int, seed=None, dataloader_kwargs=None):
    n = td.batch_size[0]
    assert n % mini_batch_size == 0, f"{n} % {mini_batch_size} != 0"
    kw = dict(dataloader_kwargs or {})
    g = torch.Generator()
    if seed is not None:
        g.manual_seed(seed)

    def gen():
        for _ in range(epochs):
            order = torch.randperm(n, generator=g) if kw.get("shuffle", True) else torch.arange(n)
            for i in range(0, n, mini_batch_size):
                yield td[order[i:i + mini_batch_size]]

    return gen()


def assert_tensordict_eq(td1: TensorDict, td2: TensorDict) -> None:
    assert set(td1.keys()) == set(td2.keys()), f"{set(td1.keys())} != {set(td2.keys())}"
    for k in td1.keys():
        a, b = td1.get(k), td2.get(k)
        assert type(a) is type(b), f"{k}: {type(a)} != {type(b)}"
        if isinstance(a, torch.Tensor):
            if a.is_nested:
                assert b.is_nested and a.size(0) == b.size(0)
                for x, y in zip(a.unbind(0), b.unbind(0)):
                    assert torch.equal(x, y), f"{k} differs"
            else:
                assert torch.equal(a, b), f"{k} differs"
        else:
            assert unwrap_non_tensor_data(a) == unwrap_non_tensor_data(b), f"{k} differs"


def get(td: TensorDict, key: str, default=None) -> Any:
    return unwrap_non_tensor_data(td.get(key, default)) if key in td else default


def get_keys(td: TensorDict, keys: Iterable[str]) -> TensorDict:
    keys = list(keys)
    missing = [k for k in keys if k not in td]
    if missing:
        raise KeyError(f"keys {missing} not found in the tensordict")
    return td.select(*keys)


def pop(td: TensorDict, key: str, default=None) -> Any:
    return unwrap_non_tensor_data(td.pop(key)) if key in td else default


def pop_keys(td: TensorDict, keys: Iterable[str]) -> TensorDict:
    out = get_keys(td, keys)
    for k in list(out.keys()):
        td.pop(k)
    return out


def pad_to_divisor(data: TensorDict, size_divisor: int):
    """Repeat leading rows until the batch divides ``size_divisor``. Returns (padded, pad_size)."""
    n = data.batch_size[0]
    pad = (-n) % size_divisor
    if pad == 0:
        return data, 0
    parts, left = [data], pad
    while left > 0:
        take = min(left, n)
        parts.append(data[torch.arange(take)])
        left -= take
    return TensorDict.cat(parts, 0), pad


def unpad(data: TensorDict, pad_size: int) -> TensorDict:
    return data[torch.arange(data.batch_size[0] - pad_size)] if pad_size else data


def contiguous(data: TensorDict) -> TensorDict:
    return data.contiguous()


def maybe_fix_3d_position_ids(data: TensorDict) -> None:
    """mrope position ids arrive as jagged [B, j, 3|4]; the model wants the rope axis first: [B, 3|4, j]."""
    if "position_ids" not in data:
        return
    p = data.get("position_ids")
    if isinstance(p, torch.Tensor) and p.is_nested:
        rows = p.unbind(0)
        if rows and rows[0].dim() == 2 and rows[0].shape[-1] in (3, 4) and rows[0].shape[0] not in (3, 4):
            data["position_ids"] = torch.nested.as_nested_tensor([r.t().contiguous() for r in rows], layout=torch.jagged)
