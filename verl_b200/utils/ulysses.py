"""Ulysses sequence parallelism: sequence-sharded activations, head-sharded attention.

Role of verl/utils/ulysses.py:1-337. Outside attention every rank of the SP group holds ``T / sp`` tokens of the
packed stream; around attention an all-to-all turns ``[T/sp, H, D]`` into ``[T, H/sp, D]`` (gather the sequence,
scatter the heads) and back. All collectives here are differentiable (the backward of an all-to-all is the inverse
all-to-all; the backward of the output all-gather is a slice scaled as in the reference, ``ulysses.py:194-240``).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

_SP_GROUP = None
_PEER_COMMS: dict = {}  # process group -> peer-memory communicator that carries the exchanges of that group


def register_peer_comm(group, comm) -> None:
    """Route the all-to-alls of ``group`` through ``comm`` (:meth:`PeerComm.all_to_all_heads`: one kernel that pulls
    straight into the output layout over NVLink) instead of ``torch.distributed``."""
    _PEER_COMMS[group] = comm


def set_ulysses_sequence_parallel_group(group) -> None:
    global _SP_GROUP
    _SP_GROUP = group


def get_ulysses_sequence_parallel_group():
    return _SP_GROUP


def get_ulysses_sequence_parallel_world_size(group=None) -> int:
    group = group if group is not None else _SP_GROUP
    return dist.get_world_size(group) if group is not None else 1


def get_ulysses_sequence_parallel_rank(group=None) -> int:
    group = group if group is not None else _SP_GROUP
    return dist.get_rank(group) if group is not None else 0


def validate_ulysses_config(num_heads: int, ulysses_sequence_size: int) -> None:
    if ulysses_sequence_size > 1 and num_heads % ulysses_sequence_size != 0:
        raise AssertionError(f"num_heads ({num_heads}) must be divisible by ulysses sequence size({ulysses_sequence_size})")


def _all_to_all(x: torch.Tensor, scatter_dim: int, gather_dim: int, group) -> torch.Tensor:
    """Split ``x`` along ``scatter_dim`` into ``sp`` parts, exchange, concatenate what arrives along ``gather_dim``."""
    sp = dist.get_world_size(group)
    if sp == 1:
        return x
    comm = _PEER_COMMS.get(group)
    if (comm is not None and x.is_cuda and x.dim() == 3 and x.element_size() == 2 and {scatter_dim, gather_dim} == {0, 1}
            and x.shape[scatter_dim] % sp == 0 and (x.shape[1] // (sp if scatter_dim == 1 else 1)) * x.shape[2] % 8 == 0):
        return comm.all_to_all_heads(x, gather_seq=(gather_dim == 0))
    parts = [t.contiguous() for t in torch.tensor_split(x, sp, dim=scatter_dim)]
    if dist.get_backend(group) == "gloo":
        # gloo has no all-to-all: gather every rank's parts and keep the ones addressed to this rank (CPU tests)
        mine = torch.stack(parts)
        everyone = [torch.empty_like(mine) for _ in range(sp)]
        dist.all_gather(everyone, mine, group=group)
        r = dist.get_rank(group)
        out = [e[r] for e in everyone]
    else:
        out = [torch.empty_like(parts[0]) for _ in range(sp)]
        dist.all_to_all(out, parts, group=group)
    return torch.cat(out, dim=gather_dim).contiguous()


class SeqAllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, group, x: torch.Tensor, scatter_dim: int, gather_dim: int):
        ctx.group, ctx.scatter_dim, ctx.gather_dim = group, scatter_dim, gather_dim
        return _all_to_all(x, scatter_dim, gather_dim, group)

    @staticmethod
    def backward(ctx, grad):
        return None, _all_to_all(grad.contiguous(), ctx.gather_dim, ctx.scatter_dim, ctx.group), None, None


def all_to_all_tensor(x: torch.Tensor, scatter_dim: int, gather_dim: int, group=None) -> torch.Tensor:
    group = group if group is not None else _SP_GROUP
    if group is None:
        return x
    return SeqAllToAll.apply(group, x, scatter_dim, gather_dim)


def gather_seq_scatter_heads(x: torch.Tensor, seq_dim: int, head_dim: int, unpadded_dim_size: int = 0, group=None) -> torch.Tensor:
    """[.., T/sp, .., H, ..] -> [.., T, .., H/sp, ..]. ``unpadded_dim_size`` trims the sequence padding afterwards."""
    group = group if group is not None else _SP_GROUP
    if group is None:
        return x
    y = all_to_all_tensor(x, head_dim, seq_dim, group)
    if unpadded_dim_size and y.shape[seq_dim] > unpadded_dim_size:
        y = y.narrow(seq_dim, 0, unpadded_dim_size)
    return y


def gather_heads_scatter_seq(x: torch.Tensor, head_dim: int, seq_dim: int, group=None) -> torch.Tensor:
    """[.., T, .., H/sp, ..] -> [.., T/sp, .., H, ..]; pads the sequence to a multiple of ``sp`` first."""
    group = group if group is not None else _SP_GROUP
    if group is None:
        return x
    sp = dist.get_world_size(group)
    pad = (-x.shape[seq_dim]) % sp
    if pad:
        shape = list(x.shape)
        shape[seq_dim] = pad
        x = torch.cat([x, x.new_zeros(shape)], dim=seq_dim)
    return all_to_all_tensor(x, seq_dim, head_dim, group)


class Gather(torch.autograd.Function):
    """All-gather along ``gather_dim``; the backward hands every rank its own slice of the gradient (optionally
    scaled by the group size, for losses that are averaged over the group afterwards)."""

    @staticmethod
    def forward(ctx, group, x: torch.Tensor, gather_dim: int, grad_scaler: bool = True):
        ctx.group, ctx.gather_dim, ctx.grad_scaler = group, gather_dim, grad_scaler
        sp = dist.get_world_size(group)
        ctx.sp, ctx.rank, ctx.part = sp, dist.get_rank(group), x.shape[gather_dim]
        parts = [torch.empty_like(x) for _ in range(sp)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=gather_dim)

    @staticmethod
    def backward(ctx, grad):
        if ctx.grad_scaler:
            grad = grad * ctx.sp
        return None, grad.narrow(ctx.gather_dim, ctx.rank * ctx.part, ctx.part).contiguous(), None, None


def gather_outputs_and_unpad(x: torch.Tensor, gather_dim: int, unpad_dim: Optional[int] = None, padding_size: int = 0,
                             grad_scaler: bool = True, group=None) -> torch.Tensor:
    group = group if group is not None else _SP_GROUP
    if group is None:
        return x
    y = Gather.apply(group, x, gather_dim, grad_scaler)
    if unpad_dim is not None and padding_size:
        y = y.narrow(unpad_dim, 0, y.shape[unpad_dim] - padding_size)
    return y


def ulysses_pad(x: torch.Tensor, dim: int, sp_size: int, value=0):
    """Pad ``dim`` to a multiple of ``sp_size``. Returns (padded, pad)."""
    pad = (-x.shape[dim]) % sp_size
    if pad == 0:
        return x, 0
    shape = list(x.shape)
    shape[dim] = pad
    return torch.cat([x, x.new_full(shape, value)], dim=dim), pad


def slice_input_tensor(x: torch.Tensor, dim: int, padding: bool = True, group=None) -> torch.Tensor:
    group = group if group is not None else _SP_GROUP
    if group is None:
        return x
    sp, r = dist.get_world_size(group), dist.get_rank(group)
    if padding:
        x, _ = ulysses_pad(x, dim, sp)
    n = x.shape[dim] // sp
    return x.narrow(dim, r * n, n).contiguous()


def ulysses_pad_and_slice_inputs(input_ids: torch.Tensor, position_ids: Optional[torch.Tensor] = None, sp_size: int = 1,
                                 group=None):
    """Packed ``input_ids`` [.., T] (and position ids) -> this rank's [.., T_pad / sp] slice. Returns
    (input_ids, position_ids, pad). Padded positions continue the last position so that RoPE stays finite."""
    if sp_size <= 1:
        return input_ids, position_ids, 0
    ids, pad = ulysses_pad(input_ids, -1, sp_size)
    pos = position_ids
    if pos is not None and pad:
        extra = torch.arange(pad, device=pos.device, dtype=pos.dtype)
        shape = list(pos.shape)
        shape[-1] = pad
        pos = torch.cat([pos, extra.expand(shape)], dim=-1)
    ids = slice_input_tensor(ids, -1, padding=False, group=group)
    if pos is not None:
        pos = slice_input_tensor(pos, -1, padding=False, group=group)
    return ids, pos, pad


def all_gather_tensor(local_tensor: torch.Tensor, gather_dim: int, group=None) -> torch.Tensor:
    """All ranks' ``local_tensor`` concatenated along ``gather_dim`` (no gradient; see :func:`gather_outputs_and_unpad`
    for the differentiable form)."""
    group = get_ulysses_sequence_parallel_group() if group is None else group
    world = dist.get_world_size(group) if group is not None else 1
    if world == 1:
        return local_tensor
    parts = [torch.empty_like(local_tensor) for _ in range(world)]
    dist.all_gather(parts, local_tensor.contiguous(), group=group)
    return torch.cat(parts, dim=gather_dim)


gather_outpus_and_unpad = gather_outputs_and_unpad  # the reference's historical spelling
