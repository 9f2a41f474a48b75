"""Tensor-parallel linear layers for inference over peer memory (sequence-parallel layout).

Role of vLLM's ``ColumnParallelLinear`` / ``RowParallelLinear`` + custom all-reduce under the reference's rollout
(verl/workers/rollout/vllm_rollout/vllm_rollout.py), in the sequence-parallel form: between the two layers of a block
the activations are split by heads / intermediate columns, outside of it by rows (tokens).

    x_rows [M / tp, K]  --all-gather-->  x [M, K]  --column-parallel GEMM-->  h [M, N / tp]
    h [M, N / tp]  --row-parallel GEMM -> reduce-scatter (one fused pass)-->  y_rows [M / tp, K]

The row-parallel layer is :meth:`PeerComm.gemm_rs`: the GEMM epilogue stores each tile into the owning rank's
receive slot over NVLink while later tiles are computed. The column-parallel layer gathers the (small) activations
with the peer-memory all-gather and runs the local GEMM. Weights are the rank's slices in the layout produced by
:mod:`verl_b200.parallel.reshard` (rows of W for column-parallel, columns of W for row-parallel).
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import ops


class ColumnParallelLinear:
    """``weight``: this rank's rows ``[N / tp, K]`` of W. Input: this rank's token rows (symmetric memory, so that
    peers can read them) or the full activations with ``gathered=True``."""

    def __init__(self, comm, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.comm, self.weight, self.bias = comm, weight, bias
        self._stage = None

    def __call__(self, x_rows: torch.Tensor, gathered: bool = False) -> torch.Tensor:
        if gathered or self.comm is None or self.comm.world == 1:
            return ops.linear(x_rows, self.weight, self.bias)
        c = self.comm
        n = x_rows.numel()
        if self._stage is None or self._stage.numel() != n:
            self._stage = c.alloc(n, x_rows.dtype, zero=False)  # collective: same shapes on every rank
        self._stage.copy_(x_rows.reshape(-1))
        full = torch.empty((c.world * x_rows.shape[0], x_rows.shape[1]), dtype=x_rows.dtype, device=x_rows.device)
        c.all_gather(full.view(-1), self._stage)
        return ops.linear(full, self.weight, self.bias)


class RowParallelLinear:
    """``weight``: this rank's columns ``[N, K / tp]`` of W. Input ``h [M, K / tp]``; output: this rank's rows
    ``[M / tp, N]`` of the summed product (+ the residual rows, if given)."""

    def __init__(self, comm, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.comm, self.weight, self.bias = comm, weight, bias

    def __call__(self, h: torch.Tensor, residual_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.comm is None or self.comm.world == 1:
            y = ops.linear(h, self.weight, self.bias)
            return y if residual_rows is None else y + residual_rows
        return self.comm.gemm_rs(h, self.weight, residual=residual_rows, bias=self.bias)


# ---------------------------------------------------------------------------------------------------------------
# Training-side tensor parallelism: the two conjugate operators of a column-parallel -> row-parallel block
# (Megatron's f / g; the reference gets them from megatron.core.tensor_parallel through its Megatron engine,
# verl/workers/engine/megatron/transformer_impl.py:57-526).
import torch.distributed as dist  # noqa: E402


class _CopyToTP(torch.autograd.Function):
    """Forward: identity on activations that are replicated over the tensor-parallel group. Backward: all-reduce, since
    every rank back-propagates only through its own slice of the following column-parallel weights."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    """Forward: all-reduce of the partial products of a row-parallel layer. Backward: identity."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def copy_to_tp_region(x: torch.Tensor, group) -> torch.Tensor:
    if group is None or dist.get_world_size(group) == 1:
        return x
    return _CopyToTP.apply(x, group)


def reduce_from_tp_region(x: torch.Tensor, group) -> torch.Tensor:
    if group is None or dist.get_world_size(group) == 1:
        return x
    return _ReduceFromTP.apply(x, group)
