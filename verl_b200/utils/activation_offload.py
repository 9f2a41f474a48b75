"""Asynchronous CPU offload of saved activations (role of verl/utils/activation_offload.py:1-558).

``enable_activation_offloading(layers)`` wraps each layer call in ``torch.autograd.graph.saved_tensors_hooks``: a
tensor saved for backward is copied to pinned host memory on a side stream right after the layer's forward (the
device copy is released once the copy is done), and copied back, again on the side stream, when backward reaches
the previous layer, so that the transfer of layer i-1 overlaps the backward compute of layer i (double buffering,
as the TE-style ``AsyncDoubleBufferGroupOffloadHandler`` of the reference). Parameters and small tensors stay on
the device.
"""

from __future__ import annotations

from typing import Iterable, Optional

import torch
from torch import nn


class _OffloadHandler:
    def __init__(self, num_groups: int, min_bytes: int = 1 << 20):
        self.num_groups = num_groups
        self.min_bytes = min_bytes
        self.stream = torch.cuda.Stream() if torch.cuda.is_available() else None
        self.cur_group = 0
        self.store: dict[int, dict[int, tuple]] = {}   # group -> tag -> (host tensor, device, event)
        self.reloaded: dict[int, dict[int, torch.Tensor]] = {}
        self._tag = 0
        self._param_ptrs: set[int] = set()

    def register_params(self, params: Iterable[torch.Tensor]):
        self._param_ptrs = {p.data_ptr() for p in params}

    # -------------------------------------------------------------- hooks
    def pack(self, t: torch.Tensor):
        if (not t.is_cuda or t.numel() * t.element_size() < self.min_bytes or t.data_ptr() in self._param_ptrs
                or isinstance(t, nn.Parameter) or not t.is_contiguous()):
            return ("keep", t)
        tag, self._tag = self._tag, self._tag + 1
        host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            host.copy_(t, non_blocking=True)
            ev = self.stream.record_event()
        t.record_stream(self.stream)  # the device copy must outlive the transfer
        self.store.setdefault(self.cur_group, {})[tag] = (host, t.device, ev)
        return ("off", self.cur_group, tag)

    def unpack(self, packed):
        if packed[0] == "keep":
            return packed[1]
        _, group, tag = packed
        if tag not in self.reloaded.get(group, {}):
            self._reload(group)
        t = self.reloaded[group].pop(tag)
        torch.cuda.current_stream().wait_stream(self.stream)
        if group - 1 >= 0 and group - 1 not in self.reloaded:
            self._reload(group - 1)  # prefetch the previous layer while this one runs its backward
        return t

    def _reload(self, group: int):
        items = self.store.pop(group, {})
        out = {}
        with torch.cuda.stream(self.stream):
            for tag, (host, dev, ev) in items.items():
                self.stream.wait_event(ev)
                out[tag] = host.to(dev, non_blocking=True)
        self.reloaded[group] = out

    def set_group(self, g: int):
        self.cur_group = g

    def reset(self):
        self.store.clear()
        self.reloaded.clear()
        self._tag = 0


class _OffloadedLayer(nn.Module):
    def __init__(self, layer: nn.Module, handler: _OffloadHandler, index: int):
        super().__init__()
        self.layer, self.handler, self.index = layer, handler, index

    def forward(self, *a, **k):
        if not torch.is_grad_enabled() or self.handler.stream is None:
            return self.layer(*a, **k)
        if self.index == 0:
            self.handler.reset()
        self.handler.set_group(self.index)
        with torch.autograd.graph.saved_tensors_hooks(self.handler.pack, self.handler.unpack):
            return self.layer(*a, **k)


def enable_activation_offloading(layers: nn.ModuleList, min_bytes: int = 1 << 20, skip_last: int = 1) -> Optional[_OffloadHandler]:
    """Wrap ``layers`` in place (all but the last ``skip_last``, whose activations are needed first in backward).
    No-op without a GPU. Returns the handler."""
    if not torch.cuda.is_available():
        return None
    handler = _OffloadHandler(len(layers), min_bytes)
    handler.register_params(p for l in layers for p in l.parameters())
    for i in range(max(0, len(layers) - skip_last)):
        layers[i] = _OffloadedLayer(layers[i], handler, i)
    return handler
