"""Contiguous per-dtype parameter buffers (role of verl/utils/memory_buffer.py:26-218): every parameter of a module
becomes a view into one flat tensor per dtype, so that weight sync moves a few large buffers instead of hundreds of
tensors."""

from __future__ import annotations

from typing import Optional

import torch
from torch import nn


class MemoryBuffer:
    def __init__(self, numel: int, numel_padded: int, dtype: torch.dtype, device=None, source: Optional[torch.Tensor] = None):
        self.numel, self.numel_padded, self.dtype = numel, numel_padded, dtype
        self.data = source if source is not None else torch.zeros(numel_padded, dtype=dtype, device=device)

    def zero(self):
        self.data.zero_()

    def get(self, shape, start_index: int) -> torch.Tensor:
        n = int(torch.Size(shape).numel())
        assert start_index + n <= self.numel, "requested tensor is out of the buffer range"
        return self.data[start_index : start_index + n].view(shape)


def calc_padded_numel(shape, dtype: torch.dtype) -> int:
    align = 128 // torch.finfo(dtype).bits if dtype.is_floating_point else 128 // torch.iinfo(dtype).bits
    n = int(torch.Size(shape).numel())
    return (n + align - 1) // align * align


def get_weight_buffer_meta_from_module(module: nn.Module) -> dict:
    return {name: {"shape": p.shape, "dtype": p.dtype} for name, p in sorted(module.named_parameters())}


def build_memory_buffer(weight_buffer_meta: dict, device=None) -> dict:
    total: dict = {}
    for _, meta in sorted(weight_buffer_meta.items()):
        total[meta["dtype"]] = total.get(meta["dtype"], 0) + calc_padded_numel(meta["shape"], meta["dtype"])
    return {dt: MemoryBuffer(n, n, dt, device) for dt, n in total.items()}


def build_memory_reference_from_module(module: nn.Module, memory_buffers: dict, maintain_weight: bool = True) -> None:
    start: dict = {dt: 0 for dt in memory_buffers}
    for _, p in sorted(module.named_parameters()):
        buf = memory_buffers[p.dtype]
        view = buf.get(p.shape, start[p.dtype])
        start[p.dtype] += calc_padded_numel(p.shape, p.dtype)
        if maintain_weight:
            view.copy_(p.data)
        p.data = view


class MemoryBufferModuleWrapper:
    """Module whose parameters live in per-dtype flat buffers."""

    def __init__(self, module: nn.Module):
        self.module = module
        self.weight_buffer_meta = get_weight_buffer_meta_from_module(module)
        device = next(module.parameters()).device
        self.memory_buffers = build_memory_buffer(self.weight_buffer_meta, device)
        build_memory_reference_from_module(module, self.memory_buffers)

    def get_memory_buffers(self) -> dict:
        return self.memory_buffers

    def get_weight_buffer_meta(self) -> dict:
        return self.weight_buffer_meta
