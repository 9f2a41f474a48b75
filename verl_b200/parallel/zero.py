"""ZeRO-3 parameter sharding with per-unit gather / recompute / reduce-scatter.

This is the engine-side replacement for torch FSDP1/FSDP2 as the reference uses them
(verl/workers/fsdp_workers.py:529-564, verl/utils/fsdp_utils.py:507-551). One *unit* is a group of
parameters that is gathered and released together (a decoder layer, the embedding, the head).

Storage (per rank, flat):
  * ``master`` fp32, ``exp_avg`` fp32, ``exp_avg_sq`` fp32, ``grad`` fp32 — 1/W of every unit
  * ``shard16`` — the working-dtype copy of ``master`` that feeds the all-gather
Every unit's padded flat parameter vector is split into W equal contiguous shards, so the
all-gather output is the flat vector itself and parameters are views into it.

With W == 1 the gathered buffer *is* ``shard16`` and the gradient buffer *is* ``grad``: no copies,
weight-gradient GEMMs accumulate straight into the optimizer's gradient (``param.main_grad``).

:func:`unit_call` runs a unit's computation under activation checkpointing: forward gathers,
computes without saving activations and releases; backward gathers again, recomputes with autograd,
back-propagates, reduce-scatters the unit's gradient into the fp32 shard and releases.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn


@dataclass
class ZeroUnit:
    name: str
    params: list  # nn.Parameter objects
    names: list  # fully-qualified names
    numel: int = 0
    padded: int = 0
    shard: int = 0
    offset: int = 0  # offset of this unit's shard inside the rank-flat buffers
    offsets: list = field(default_factory=list)  # per-parameter offsets inside the unit's flat vector
    shapes: list = field(default_factory=list)  # parameter shapes (parameters are emptied while released)
    numels: list = field(default_factory=list)
    full: Optional[torch.Tensor] = None  # gathered working-dtype buffer (None when released)
    full_grad: Optional[torch.Tensor] = None  # unit-sized fp32 gradient buffer during backward (W > 1)
    gather_count: int = 0
    index: int = 0  # position in ZeroShardedParams.units
    ready: Optional[object] = None  # event of the gather that fills ``full`` on the communication stream
    grad_seq: int = -1  # sequence number of this backward's gradient buffer / reduce-scatter
    # Expert parallelism: a unit of stacked expert matrices [E, ...] whose rank-r shard is exactly experts
    # [r E / W, (r + 1) E / W). It is never gathered for compute: the parameters are permanent views of this rank's
    # shard (shape [E / W, ...]) and their gradients accumulate straight into this rank's gradient shard, because the
    # tokens routed to these experts are sent here. Storage, optimizer, checkpoints and the train -> rollout reshard
    # see an ordinary sharded unit.
    local: bool = False


class ZeroShardedParams:
    """Owns the sharded state of a model and the gather / reduce-scatter mechanics."""

    def __init__(self, units: Sequence[tuple[str, nn.Module | list]], *, group=None, work_dtype=torch.bfloat16,
                 device="cuda", trainable: bool = True, align: int = 256, comm=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.work_dtype = work_dtype
        self.device = torch.device(device)
        self.trainable = trainable
        # frozen parameters inside a differentiable graph (LoRA base weights): unit calls run under autograd so that
        # gradients reach the inputs and the tensors captured by the call, but nothing is kept for the parameters
        self.frozen_grad = False
        self.comm = comm  # optional accelerated collectives (peer-memory kernels); falls back to torch.distributed
        self.units: list[ZeroUnit] = []
        self._anchor = None
        seen: set[int] = set()
        off = 0
        for spec in units:
            name, mod = spec[0], spec[1]
            opts = spec[2] if len(spec) > 2 else {}
            named = list(mod.named_parameters()) if isinstance(mod, nn.Module) else list(mod)
            named = [(n, p) for n, p in named if id(p) not in seen]
            seen.update(id(p) for _, p in named)
            u = ZeroUnit(name=name, params=[p for _, p in named], names=[f"{name}.{n}" if name else n for n, _ in named])
            cur = 0
            for p in u.params:
                u.offsets.append(cur)
                u.shapes.append(tuple(p.shape))
                u.numels.append(p.numel())
                cur += (p.numel() + 7) // 8 * 8  # keep every tensor 16-byte aligned in bf16
            u.numel = cur
            quantum = align * self.world
            u.padded = (cur + quantum - 1) // quantum * quantum
            if opts.get("local") and self.world > 1:
                p0 = u.params[0]
                ok = (len(u.params) == 1 and p0.dim() >= 2 and p0.shape[0] % self.world == 0
                      and (p0.numel() // self.world) % 8 == 0)
                if not ok:
                    raise ValueError(f"expert-parallel unit {name}: one stacked tensor [E, ...] with E divisible by the "
                                     f"{self.world} ranks and 16-byte aligned expert slices is required")
                u.local = True
                u.padded = p0.numel()
            u.shard = u.padded // self.world
            u.offset = off
            off += u.shard
            u.index = len(self.units)
            self.units.append(u)
        self.total_shard = off
        # Gathers of the next unit and reduce-scatters of the previous one run on their own stream, under the
        # compute of the current unit (peer-memory collectives only).
        self.comm_stream = torch.cuda.Stream(device=self.device) if (comm is not None and self.world > 1) else None
        self._rs_done: dict = {}
        self._grad_seq = 0
        dev = self.device
        if comm is not None and self.world > 1:
            # peers read this shard directly over NVLink: it lives in symmetric memory
            self.shard16 = comm.alloc(off, work_dtype)
            if trainable:
                comm.reserve_grad_buffers(max(u.padded for u in self.units), count=3)
        else:
            self.shard16 = torch.zeros(off, dtype=work_dtype, device=dev)
        if trainable:
            self.master = torch.zeros(off, dtype=torch.float32, device=dev)
            self.exp_avg = torch.zeros(off, dtype=torch.float32, device=dev)
            self.exp_avg_sq = torch.zeros(off, dtype=torch.float32, device=dev)
            self.grad = torch.zeros(off, dtype=torch.float32, device=dev)
        else:
            self.master = self.exp_avg = self.exp_avg_sq = self.grad = None
        self._load_from_params()
        if self.world == 1:
            for u in self.units:
                self._bind(u, self.shard16[u.offset : u.offset + u.shard],
                           self.grad[u.offset : u.offset + u.shard] if trainable else None)
                u.full = self.shard16[u.offset : u.offset + u.shard]
        else:
            for u in self.units:
                if u.local:
                    self._bind_local(u)
                else:
                    self._unbind(u)

    # ------------------------------------------------------------- initial load
    @torch.no_grad()
    def _load_from_params(self):
        """Copy the module's current parameter values (identical on all ranks) into this rank's shards."""
        for u in self.units:
            lo, hi = self.rank * u.shard, (self.rank + 1) * u.shard
            for p, o in zip(u.params, u.offsets):
                s, e = max(o, lo), min(o + p.numel(), hi)
                if s >= e:
                    continue
                src = p.detach().reshape(-1)[s - o : e - o]
                dst = slice(u.offset + s - lo, u.offset + e - lo)
                if self.trainable:
                    self.master[dst].copy_(src.float())
                self.shard16[dst].copy_(src.to(self.work_dtype))

    def _bind(self, u: ZeroUnit, full: torch.Tensor, full_grad: Optional[torch.Tensor]):
        for p, o, shape, n in zip(u.params, u.offsets, u.shapes, u.numels):
            p.data = full[o : o + n].view(shape)
            if full_grad is not None and p.requires_grad:
                p.main_grad = full_grad[o : o + n].view(shape)

    def _bind_local(self, u: ZeroUnit):
        """Expert-parallel unit: the parameter becomes this rank's experts, a view of the shard."""
        p, shape = u.params[0], u.shapes[0]
        local_shape = (shape[0] // self.world,) + tuple(shape[1:])
        p.data = self.shard16[u.offset : u.offset + u.shard].view(local_shape)
        if self.trainable and p.requires_grad:
            p.main_grad = self.grad[u.offset : u.offset + u.shard].view(local_shape)

    def _unbind(self, u: ZeroUnit):
        empty = torch.empty(0, dtype=self.work_dtype, device=self.device)
        for p in u.params:
            p.data = empty
            if hasattr(p, "main_grad"):
                del p.main_grad

    # ---------------------------------------------------------- gather / release
    def _issue_gather(self, u: ZeroUnit):
        """Start the all-gather of ``u`` (on the communication stream when there is one)."""
        full = torch.empty(u.padded, dtype=self.work_dtype, device=self.device)
        src = self.shard16[u.offset : u.offset + u.shard]
        if self.comm_stream is not None:
            main = torch.cuda.current_stream(self.device)
            self.comm_stream.wait_stream(main)  # the buffer is free and this rank's shard is final
            with torch.cuda.stream(self.comm_stream):
                self.comm.all_gather(full, src)
                u.ready = self.comm_stream.record_event()
        elif self.comm is not None:
            self.comm.all_gather(full, src)
        else:
            dist.all_gather_into_tensor(full, src, group=self.group)
        u.full = full

    def _next_grad_buffer(self, u: ZeroUnit) -> torch.Tensor:
        """Symmetric fp32 buffer for the unit's gradients. Three buffers rotate: peers read buffer n during
        reduce-scatter n, and this rank knows they are done once its own reduce-scatter n+1 has completed
        (its entry barrier proves that every peer has started n+1, hence finished n)."""
        n = self._grad_seq
        self._grad_seq += 1
        u.grad_seq = n
        ev = self._rs_done.pop(n - 2, None)
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)
        return self.comm.grad_buffer(u.padded)

    def wait_comm(self):
        """Make the current stream wait for every collective issued on the communication stream."""
        if self.comm_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
            self._rs_done.clear()

    def gather(self, u: ZeroUnit, for_backward: bool = False, prefetch: bool = True):
        u.gather_count += 1
        if self.world == 1 or u.local:
            return
        if u.full is None:
            self._issue_gather(u)
        if u.ready is not None:
            torch.cuda.current_stream(self.device).wait_event(u.ready)
            u.ready = None
        if prefetch and self.comm_stream is not None:
            j = u.index + (-1 if for_backward else 1)
            if 0 <= j < len(self.units) and self.units[j].full is None and not self.units[j].local:
                self._issue_gather(self.units[j])
        if for_backward and self.trainable and u.full_grad is None:
            if self.comm is not None:
                u.full_grad = self._next_grad_buffer(u)
            else:
                u.full_grad = torch.zeros(u.padded, dtype=torch.float32, device=self.device)
        self._bind(u, u.full, u.full_grad if for_backward else None)

    def release(self, u: ZeroUnit):
        u.gather_count -= 1
        if self.world == 1 or u.gather_count > 0 or u.local:
            return
        self._unbind(u)
        u.full = None
        u.full_grad = None

    def fold_param_grads(self, u: ZeroUnit):
        """Gradients that autograd left in ``p.grad`` (ops without a fused accumulate) go to ``main_grad``."""
        for p in u.params:
            if p.grad is not None:
                if hasattr(p, "main_grad"):
                    p.main_grad.add_(p.grad.float())
                p.grad = None

    def reduce_grads(self, u: ZeroUnit):
        """Sum the unit's gradient over ranks and add this rank's slice into the fp32 gradient shard."""
        self.fold_param_grads(u)
        if self.world == 1 or not self.trainable or u.full_grad is None or u.local:
            return
        dst = self.grad[u.offset : u.offset + u.shard]
        if self.comm_stream is not None:
            self.comm_stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.comm_stream):
                self.comm.reduce_scatter_add(dst, u.full_grad)
                self._rs_done[u.grad_seq] = self.comm_stream.record_event()
        elif self.comm is not None:
            self.comm.reduce_scatter_add(dst, u.full_grad)
        elif dist.get_backend(self.group) == "gloo":
            dist.all_reduce(u.full_grad, group=self.group)
            dst.add_(u.full_grad[self.rank * u.shard : (self.rank + 1) * u.shard])
        else:
            tmp = torch.empty(u.shard, dtype=torch.float32, device=self.device)
            dist.reduce_scatter_tensor(tmp, u.full_grad, group=self.group)
            dst.add_(tmp)
        u.full_grad = None

    # ------------------------------------------------------------ whole-model views
    def gather_all(self):
        for u in self.units:
            self.gather(u)

    def release_all(self):
        for u in self.units:
            self.release(u)

    def full_tensor(self, u: ZeroUnit, idx: int, dtype=None) -> torch.Tensor:
        """One full parameter of a (currently gathered) unit."""
        o = u.offsets[idx]
        t = u.full[o : o + u.numels[idx]].view(u.shapes[idx])
        return t if dtype is None else t.to(dtype)

    def named_full_tensors(self, dtype=None):
        """Generator of (name, full tensor), gathering one unit at a time (weight export / sync).
        Role of ``get_per_tensor_param`` (verl/workers/engine/fsdp/transformer_impl.py:635-671)."""
        for u in self.units:
            if u.local and self.world > 1:  # expert-parallel unit: gathered for export only
                full = torch.empty(u.padded, dtype=self.work_dtype, device=self.device)
                dist.all_gather_into_tensor(full, self.shard16[u.offset : u.offset + u.shard].contiguous(), group=self.group)
                t = full.view(u.shapes[0])
                yield u.names[0], (t if dtype is None else t.to(dtype))
                continue
            self.gather(u)
            try:
                for i, name in enumerate(u.names):
                    yield name, self.full_tensor(u, i, dtype)
            finally:
                self.release(u)

    @torch.no_grad()
    def load_full_state(self, state: dict[str, torch.Tensor], strict: bool = True):
        """Set parameters (and fp32 masters) from full tensors keyed by parameter name."""
        missing = []
        for u in self.units:
            lo, hi = self.rank * u.shard, (self.rank + 1) * u.shard
            for name, n, o in zip(u.names, u.numels, u.offsets):
                if name not in state:
                    missing.append(name)
                    continue
                s, e = max(o, lo), min(o + n, hi)
                if s >= e:
                    continue
                src = state[name].reshape(-1)[s - o : e - o].to(self.device)
                dst = slice(u.offset + s - lo, u.offset + e - lo)
                if self.trainable:
                    self.master[dst].copy_(src.float())
                self.shard16[dst].copy_(src.to(self.work_dtype))
        if strict and missing:
            raise KeyError(f"missing parameters: {missing[:5]}{'...' if len(missing) > 5 else ''}")
        return missing

    def zero_grad(self):
        if self.trainable:
            self.wait_comm()
            self.grad.zero_()

    # ------------------------------------------------------------ sharded state io
    def shard_state(self) -> dict:
        """This rank's shard of model / optimizer state plus the layout needed to re-assemble it."""
        layout = [{"name": u.name, "names": u.names, "shapes": list(u.shapes), "offsets": u.offsets,
                   "numel": u.numel, "padded": u.padded, "shard": u.shard, "offset": u.offset} for u in self.units]
        out = {"layout": layout, "world_size": self.world, "rank": self.rank, "shard16": self.shard16.cpu()}
        if self.trainable:
            out.update(master=self.master.cpu(), exp_avg=self.exp_avg.cpu(), exp_avg_sq=self.exp_avg_sq.cpu())
        return out

    @torch.no_grad()
    def load_shard_state(self, st: dict, load_optimizer: bool = True):
        assert st["world_size"] == self.world, f"checkpoint world size {st['world_size']} != {self.world}"
        self.shard16.copy_(st["shard16"].to(self.device))
        if self.trainable and "master" in st:
            self.master.copy_(st["master"].to(self.device))
            if load_optimizer:
                self.exp_avg.copy_(st["exp_avg"].to(self.device))
                self.exp_avg_sq.copy_(st["exp_avg_sq"].to(self.device))

    # ------------------------------------------------------------------ offload
    def offload(self, params: bool = True, optimizer: bool = True):
        """Move shards to pinned host memory (param_offload / optimizer_offload)."""
        def to_host(t):
            if t is None or not t.is_cuda:
                return t
            h = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
            h.copy_(t, non_blocking=True)
            return h

        if params and self.world > 1 and self.comm is None:
            for u in self.units:
                if u.local:
                    self._unbind(u)
            self.shard16 = to_host(self.shard16)
        if optimizer and self.trainable:
            self.master, self.exp_avg, self.exp_avg_sq = map(to_host, (self.master, self.exp_avg, self.exp_avg_sq))
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()

    def reload(self):
        dev = self.device
        for name in ("shard16", "master", "exp_avg", "exp_avg_sq"):
            t = getattr(self, name)
            if t is not None and t.device != dev:
                setattr(self, name, t.to(dev, non_blocking=True))
        for u in self.units:
            if u.local and self.world > 1:
                self._bind_local(u)

    def fold_local_units(self):
        """Expert-parallel units are outside the per-layer gather / reduce cycle: gradients that autograd left in
        ``p.grad`` (ops without a fused accumulate) are added to the gradient shard here, before the optimizer step."""
        for u in self.units:
            if u.local:
                self.fold_param_grads(u)


class _UnitFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, zero: ZeroShardedParams, unit: ZeroUnit, fn: Callable, mask: tuple, *tensors):
        ctx.zero, ctx.unit, ctx.fn, ctx.mask = zero, unit, fn, mask
        tensors = tensors[:-1]  # the last input is the graph anchor (see unit_call)
        zero.gather(unit)
        try:
            with torch.no_grad():
                outs = fn(*_expand(mask, tensors))
        finally:
            zero.release(unit)
        ctx.save_for_backward(*tensors)
        ctx.single = not isinstance(outs, tuple)
        return outs

    @staticmethod
    def backward(ctx, *grads):
        zero, unit = ctx.zero, ctx.unit
        inputs = [t.detach().requires_grad_(t.is_floating_point()) for t in ctx.saved_tensors]
        zero.gather(unit, for_backward=True)
        try:
            with torch.enable_grad():
                outs = ctx.fn(*_expand(ctx.mask, inputs))
            outs = (outs,) if ctx.single else outs
            pairs = [(o, g) for o, g in zip(outs, grads) if g is not None and isinstance(o, torch.Tensor) and o.requires_grad]
            if pairs:
                torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
            zero.reduce_grads(unit)
        finally:
            zero.release(unit)
        return (None, None, None, None) + tuple(t.grad if t.requires_grad else None for t in inputs) + (None,)


class _UnitFnKeep(torch.autograd.Function):
    """Like :class:`_UnitFn` but the unit's activations are kept: the forward records the unit's autograd graph and
    the backward runs it (no recomputation) after gathering the parameters again. The graph refers to the unit's
    ``Parameter`` objects, whose storage is re-bound by every gather, so it reads the re-gathered weights."""

    @staticmethod
    def forward(ctx, zero: ZeroShardedParams, unit: ZeroUnit, fn: Callable, mask: tuple, *tensors):
        ctx.zero, ctx.unit = zero, unit
        inputs = [t.detach().requires_grad_(t.is_floating_point()) for t in tensors[:-1]]
        zero.gather(unit)
        try:
            with torch.enable_grad():
                outs = fn(*_expand(mask, inputs))
        finally:
            zero.release(unit)
        ctx.single = not isinstance(outs, tuple)
        ctx.inputs, ctx.outs = inputs, ((outs,) if ctx.single else outs)
        det = tuple(o.detach() if isinstance(o, torch.Tensor) else o for o in ctx.outs)
        return det[0] if ctx.single else det

    @staticmethod
    def backward(ctx, *grads):
        zero, unit = ctx.zero, ctx.unit
        inputs, outs = ctx.inputs, ctx.outs
        ctx.inputs = ctx.outs = None
        zero.gather(unit, for_backward=True)
        try:
            pairs = [(o, g) for o, g in zip(outs, grads) if g is not None and isinstance(o, torch.Tensor) and o.requires_grad]
            if pairs:
                torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
            zero.reduce_grads(unit)
        finally:
            zero.release(unit)
        return (None, None, None, None) + tuple(t.grad if t.requires_grad else None for t in inputs) + (None,)


def _expand(mask, tensors):
    it = iter(tensors)
    return [next(it) if m else None for m in mask]


def unit_call(zero: ZeroShardedParams, unit: ZeroUnit, fn: Callable, *args, keep_activations: bool = False):
    """Run ``fn(*args)`` (tensor or None arguments) with the unit's parameters gathered. With grad enabled
    the call is checkpointed: activations are recomputed in backward (or kept, with ``keep_activations``), and the
    unit's gradients are reduce-scattered right after its backward."""
    mask = tuple(a is not None for a in args)
    tensors = [a for a in args if a is not None]
    if torch.is_grad_enabled() and (zero.trainable or zero.frozen_grad):
        # a unit whose inputs carry no gradient (the embedding: integer ids) must still get a backward
        # call for its parameters, so every call is anchored on a scalar that requires grad
        if zero._anchor is None:
            zero._anchor = torch.zeros(1, device=zero.device, requires_grad=True)
        return (_UnitFnKeep if keep_activations else _UnitFn).apply(zero, unit, fn, mask, *tensors, zero._anchor)
    zero.gather(unit)
    try:
        with torch.no_grad():
            return fn(*args)
    finally:
        zero.release(unit)
