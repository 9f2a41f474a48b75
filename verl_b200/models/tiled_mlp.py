"""Sequence-tiled MLP (verl/models/transformers/tiled_mlp.py): run the gate/up -> SwiGLU -> down block over row
shards of the packed token stream and recompute each shard in the backward, so the ``[T, 2 * intermediate]``
activation never exists for more than ``T / num_shards`` rows. Useful for very long packed streams; with 180 GB per
GPU the default is off (``model.tiled_mlp.enabled``)."""

from __future__ import annotations

import torch
import torch.nn as nn


class _TiledMLPFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, mlp, num_shards: int, x: torch.Tensor, *params):
        ctx.mlp, ctx.num_shards, ctx.params = mlp, num_shards, list(params)
        ctx.save_for_backward(x)
        with torch.no_grad():
            return torch.cat([mlp(c) for c in torch.tensor_split(x, num_shards, dim=0)], dim=0)

    @staticmethod
    def backward(ctx, grad_out):
        (x,) = ctx.saved_tensors
        params = ctx.params
        dx = torch.empty_like(x)
        grads = [None] * len(params)
        bounds = torch.tensor_split(torch.arange(x.shape[0]), ctx.num_shards)
        for b in bounds:
            if b.numel() == 0:
                continue
            lo, hi = int(b[0]), int(b[-1]) + 1
            xc = x[lo:hi].detach().requires_grad_(True)
            with torch.enable_grad():
                yc = ctx.mlp(xc)
            g = torch.autograd.grad(yc, [xc] + params, grad_out[lo:hi], allow_unused=True)
            dx[lo:hi] = g[0]
            for i, gi in enumerate(g[1:]):
                if gi is not None:
                    grads[i] = gi if grads[i] is None else grads[i] + gi
        return (None, None, dx, *grads)


class TiledMLP(nn.Module):
    """Wraps an MLP module ``[T, H] -> [T, H]``; parameters stay those of the wrapped module."""

    def __init__(self, mlp: nn.Module, num_shards: int = 4):
        super().__init__()
        self.mlp, self.num_shards = mlp, int(num_shards)

    def forward(self, x):
        return tiled_call(self.mlp, list(self.mlp.parameters()), self.num_shards, x)


def tiled_call(fn, params, num_shards: int, x: torch.Tensor) -> torch.Tensor:
    """``fn(x)`` over ``num_shards`` row shards with per-shard recomputation; ``params`` are the tensors ``fn`` reads."""
    if num_shards <= 1 or not torch.is_grad_enabled() or x.shape[0] < num_shards:
        return fn(x)
    return _TiledMLPFn.apply(fn, num_shards, x, *params)


def apply_tiled_mlp(model: nn.Module, num_shards: int = 4) -> int:
    """Switch every dense MLP of a :class:`CausalLM` to the tiled path (parameter names do not change). Returns how
    many layers were switched."""
    from .transformer import DenseMLP

    n = 0
    for layer in getattr(model, "layers", []):
        if isinstance(getattr(layer, "mlp", None), DenseMLP):
            layer.mlp.tile_shards = int(num_shards)
            n += 1
    return n
