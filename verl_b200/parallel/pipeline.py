"""Pipeline parallelism: point-to-point transfer of the residual stream between consecutive stages as autograd
functions (send in the forward = receive of the gradient in the backward, and the reverse).

The reference gets pipeline (and virtual pipeline) schedules from Megatron-core
(verl/workers/engine/megatron/transformer_impl.py:496-521 ``get_forward_backward_func``); its transfers are NCCL
point-to-point calls. Here a stage sends ONE tensor per micro-batch: ``hidden + residual`` (the next stage's first
RMSNorm re-creates both). Transfers are ``torch.distributed`` send / recv on the default group (NCCL p2p on CUDA, gloo on
CPU); micro-batches of a batch are pipelined by :meth:`NativeEngine.forward_backward_batch` (all forwards, then all
backwards, in one fixed order on every stage).
"""

from __future__ import annotations

import torch
import torch.distributed as dist


class _PipeSend(torch.autograd.Function):
    """Forward: send ``x`` to the next stage; returns a scalar zero that keeps the graph alive. Backward: receive the
    gradient of ``x`` from the next stage (whatever gradient arrives for the scalar is ignored)."""

    @staticmethod
    def forward(ctx, x, dst: int):
        x = x.contiguous()
        ctx.dst, ctx.shape, ctx.dtype, ctx.device = dst, x.shape, x.dtype, x.device
        dist.send(x, dst=dst)
        return x.new_zeros(())

    @staticmethod
    def backward(ctx, g):
        grad = torch.empty(ctx.shape, dtype=ctx.dtype, device=ctx.device)
        dist.recv(grad, src=ctx.dst)
        return grad, None


class _PipeRecv(torch.autograd.Function):
    """Forward: receive a tensor of the given shape from the previous stage (``anchor`` is a dummy input that requires
    grad so that the backward runs). Backward: send the gradient back."""

    @staticmethod
    def forward(ctx, anchor, src: int, shape, dtype, device):
        ctx.src = src
        buf = torch.empty(shape, dtype=dtype, device=device)
        dist.recv(buf, src=src)
        return buf

    @staticmethod
    def backward(ctx, g):
        dist.send(g.contiguous(), dst=ctx.src)
        return torch.zeros((), dtype=g.dtype, device=g.device), None, None, None, None


def pipe_send(x: torch.Tensor, dst: int) -> torch.Tensor:
    if torch.is_grad_enabled() and x.requires_grad:
        return _PipeSend.apply(x, dst)
    dist.send(x.contiguous(), dst=dst)
    return x.new_zeros(())


def pipe_recv(src: int, shape, dtype, device, need_grad: bool) -> torch.Tensor:
    if need_grad and torch.is_grad_enabled():
        anchor = torch.zeros((), dtype=torch.float32, device=device, requires_grad=True)
        return _PipeRecv.apply(anchor, src, tuple(shape), dtype, device)
    buf = torch.empty(tuple(shape), dtype=dtype, device=device)
    dist.recv(buf, src=src)
    return buf


def stage_layers(num_layers: int, pp_size: int, pp_rank: int) -> tuple[int, int]:
    """Contiguous, near-equal split of the decoder layers (earlier stages take the remainder)."""
    base, rem = divmod(num_layers, pp_size)
    lo = pp_rank * base + min(pp_rank, rem)
    return lo, lo + base + (1 if pp_rank < rem else 0)
