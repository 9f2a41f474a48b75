"""Model ops (RMSNorm, RoPE, SwiGLU, embedding) as autograd functions over the native kernels.

CUDA tensors always go to the hand-written kernels (bf16 storage, fp32 math); CPU tensors
use an equivalent plain-torch path so the same model code runs in the CPU test tier.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib


# --------------------------------------------------------------------------- RMSNorm
def _rmsnorm_ref(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


class _RMSNormFn(torch.autograd.Function):
    """y = rmsnorm(x + residual) * w; also returns the new residual stream (x + residual)."""

    @staticmethod
    def forward(ctx, x, residual, weight, eps):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        if residual is not None:
            r2 = residual.reshape(-1, H)
            h = torch.empty_like(x2)
            rc = _lib.fn("vb_rmsnorm_fwd")(x2.data_ptr(), r2.data_ptr(), weight.data_ptr(), y.data_ptr(), h.data_ptr(),
                                           rstd.data_ptr(), rows, H, eps, _lib.stream())
        else:
            h = x2
            rc = _lib.fn("vb_rmsnorm_fwd")(x2.data_ptr(), None, weight.data_ptr(), y.data_ptr(), None,
                                           rstd.data_ptr(), rows, H, eps, _lib.stream())
        _lib.check(rc, "vb_rmsnorm_fwd")
        ctx.save_for_backward(h, weight, rstd)
        ctx.has_res = residual is not None
        ctx.shape = x.shape
        if residual is not None:
            return y.reshape(x.shape), h.reshape(x.shape)
        return y.reshape(x.shape), x

    @staticmethod
    def backward(ctx, dy, dh):
        h, weight, rstd = ctx.saved_tensors
        H = h.shape[-1]
        rows = h.shape[0]
        dy2 = dy.reshape(-1, H).contiguous()
        dres = dh.reshape(-1, H).contiguous() if dh is not None else None
        dx = torch.empty_like(h)
        parts = _lib.fn("vb_rmsnorm_bwd_parts")(rows)
        dwp = torch.empty(parts, H, dtype=torch.float32, device=h.device)
        main_grad = getattr(weight, "main_grad", None)
        if main_grad is not None:
            dw_buf, acc = main_grad, 1
        else:
            dw_buf, acc = torch.empty(H, dtype=torch.float32, device=h.device), 0
        rc = _lib.fn("vb_rmsnorm_bwd")(dy2.data_ptr(), h.data_ptr(), weight.data_ptr(), rstd.data_ptr(),
                                       _lib.ptr(dres), dx.data_ptr(), dwp.data_ptr(), dw_buf.data_ptr(), acc, rows, H,
                                       _lib.stream())
        _lib.check(rc, "vb_rmsnorm_bwd")
        dx = dx.reshape(ctx.shape)
        dw = None if main_grad is not None else dw_buf.to(weight.dtype)
        # the gradient of the residual stream flows to both x and residual
        return dx, (dx if ctx.has_res else None), dw, None


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, residual: torch.Tensor | None = None):
    """Returns ``(normed, new_residual)`` where ``new_residual = x + residual`` (or ``x``)."""
    if x.is_cuda:
        if residual is None and not torch.is_grad_enabled():
            pass
        return _RMSNormFn.apply(x.contiguous(), None if residual is None else residual.contiguous(), weight, eps)
    h = x if residual is None else x + residual
    return _rmsnorm_ref(h, weight, eps), h


# ------------------------------------------------------------------------------ RoPE
_rope_cache: dict = {}


def rope_tables(head_dim: int, max_pos: int, theta: float, device, scaling: dict | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """cos / sin tables [max_pos, head_dim / 2]. ``scaling``: the HF ``rope_scaling`` / ``rope_parameters`` dict;
    ``llama3`` (frequencies below the low-frequency cut divided by ``factor``, a smooth blend up to the high-frequency
    cut: Llama 3.1+, Apertus) and ``linear`` (all frequencies divided by ``factor``) are implemented."""
    kind = (scaling or {}).get("rope_type") or (scaling or {}).get("type") or "default"
    key = (head_dim, max_pos, float(theta), str(device), kind, tuple(sorted((k, str(v)) for k, v in (scaling or {}).items())))
    if key not in _rope_cache:
        inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
        if kind == "llama3":
            import math

            factor = float(scaling.get("factor", 8.0))
            lo, hi = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
            orig = float(scaling.get("original_max_position_embeddings", 8192))
            wavelen = 2 * math.pi / inv
            smooth = ((orig / wavelen - lo) / (hi - lo)).clamp(0.0, 1.0)
            blended = (1 - smooth) * inv / factor + smooth * inv
            inv = torch.where(wavelen > orig / lo, inv / factor, torch.where(wavelen < orig / hi, inv, blended))
        elif kind == "linear":
            inv = inv / float(scaling.get("factor", 1.0))
        elif kind not in ("default", "mrope"):
            raise NotImplementedError(f"rope scaling type {kind!r} is not implemented")
        ang = torch.arange(max_pos, dtype=torch.float32, device=device)[:, None] * inv[None]
        _rope_cache[key] = (ang.cos().contiguous(), ang.sin().contiguous())
    return _rope_cache[key]


def _rope_ref(t, pos, cos_t, sin_t, n_heads, D, sign=1.0):
    T = t.shape[0]
    tf = t.float().reshape(T, n_heads, D)
    c = cos_t[pos][:, None, :]
    s = sin_t[pos][:, None, :] * sign
    a, b = tf[..., : D // 2], tf[..., D // 2 :]
    return torch.cat([a * c - b * s, b * c + a * s], -1).reshape(T, n_heads * D).to(t.dtype)


def _mrope_cos_sin(pos3, cos_t, sin_t, sections, interleaved: bool = False):
    """Per-token cos / sin [T, D/2] of multimodal RoPE: frequency j follows the temporal / height / width position
    according to ``sections`` (numbers of frequencies per axis): three consecutive runs (Qwen2-VL), or, ``interleaved``
    (Qwen3-VL), frequency j follows height if j % 3 == 1 and j < 3 * sections[1], width if j % 3 == 2 and
    j < 3 * sections[2], the temporal position otherwise (T H W T H W ... T T)."""
    half = cos_t.shape[1]
    if interleaved:
        j = torch.arange(half, device=pos3.device)
        axis = torch.zeros(half, dtype=torch.long, device=pos3.device)
        axis[(j % 3 == 1) & (j < 3 * int(sections[1]))] = 1
        axis[(j % 3 == 2) & (j < 3 * int(sections[2]))] = 2
    else:
        axis = torch.repeat_interleave(torch.arange(3, device=pos3.device), torch.tensor(list(sections), device=pos3.device))
    axis = axis[:half]
    j = torch.arange(half, device=pos3.device)
    p = pos3[axis]                      # [half, T]: the position each frequency uses
    return cos_t[p, j[:, None]].t().contiguous(), sin_t[p, j[:, None]].t().contiguous()


class _RopeFn(torch.autograd.Function):
    """In-place rotary embedding on the q and k slices of a packed qkv activation [T, (Hq+2Hk)*D]. ``sections``
    (multimodal RoPE) makes ``pos`` a [3, T] tensor of temporal / height / width positions."""

    @staticmethod
    def _run(qkv, pos, cos_t, sin_t, Hq, Hk, D, sections, backward):
        T = qkv.shape[0]
        q = qkv[:, : Hq * D]
        k = qkv[:, Hq * D : (Hq + Hk) * D]
        if sections is None:
            rc = _lib.fn("vb_rope")(q.data_ptr(), k.data_ptr(), qkv.stride(0), qkv.stride(0), pos.data_ptr(),
                                    cos_t.data_ptr(), sin_t.data_ptr(), T, Hq, Hk, D, backward, _lib.stream())
        else:
            rc = _lib.fn("vb_mrope")(q.data_ptr(), k.data_ptr(), qkv.stride(0), qkv.stride(0), pos.data_ptr(),
                                     cos_t.data_ptr(), sin_t.data_ptr(), T, Hq, Hk, D, int(sections[0]), int(sections[1]),
                                     backward, _lib.stream())
        _lib.check(rc, "vb_rope")

    @staticmethod
    def forward(ctx, qkv, pos, cos_t, sin_t, Hq, Hk, D, sections):
        _RopeFn._run(qkv, pos, cos_t, sin_t, Hq, Hk, D, sections, 0)
        ctx.save_for_backward(pos, cos_t, sin_t)
        ctx.dims = (Hq, Hk, D, sections)
        ctx.mark_dirty(qkv)
        return qkv

    @staticmethod
    def backward(ctx, dqkv):
        pos, cos_t, sin_t = ctx.saved_tensors
        Hq, Hk, D, sections = ctx.dims
        dqkv = dqkv.contiguous().clone() if not dqkv.is_contiguous() else dqkv.clone()
        _RopeFn._run(dqkv, pos, cos_t, sin_t, Hq, Hk, D, sections, 1)
        return dqkv, None, None, None, None, None, None, None


def rope_qkv(qkv: torch.Tensor, pos: torch.Tensor, cos_t: torch.Tensor, sin_t: torch.Tensor, Hq: int, Hk: int, D: int,
             mrope_section=None, mrope_interleaved: bool = False):
    """Apply rotate-half RoPE to the q and k parts of packed ``qkv`` ([T, (Hq+2Hk)*D]); v is untouched. With
    ``mrope_section = (t, h, w)`` (frequencies per axis, sum D / 2) ``pos`` is ``[3, T]`` (multimodal RoPE of the
    Qwen2-VL family, verl/models/transformers/qwen2_vl.py; ``mrope_interleaved``: the layout of Qwen3-VL,
    verl/models/transformers/qwen3_vl.py, which takes the per-token-table path below: the kernel knows the sectioned
    layout only)."""
    if pos.dim() == 2 and mrope_section is None:
        pos = pos[0]
    if pos.dim() == 1:
        mrope_section = None
    if qkv.is_cuda and (mrope_section is None or
                        (not mrope_interleaved and all(int(x) % 8 == 0 for x in mrope_section[:2]))):
        return _RopeFn.apply(qkv, pos.contiguous(), cos_t, sin_t, Hq, Hk, D,
                             None if mrope_section is None else tuple(int(x) for x in mrope_section))
    if mrope_section is not None:
        c, s_ = _mrope_cos_sin(pos, cos_t, sin_t, mrope_section, mrope_interleaved)
        q = _rope_apply(qkv[:, : Hq * D], c, s_, Hq, D)
        k = _rope_apply(qkv[:, Hq * D : (Hq + Hk) * D], c, s_, Hk, D)
        return torch.cat([q, k, qkv[:, (Hq + Hk) * D :]], dim=-1)
    q = _rope_ref(qkv[:, : Hq * D], pos, cos_t, sin_t, Hq, D)
    k = _rope_ref(qkv[:, Hq * D : (Hq + Hk) * D], pos, cos_t, sin_t, Hk, D)
    return torch.cat([q, k, qkv[:, (Hq + Hk) * D :]], dim=-1)


def _rope_apply(t, c, s_, n_heads, D):
    """Rotate-half with per-token cos / sin [T, D/2]."""
    T = t.shape[0]
    tf = t.float().reshape(T, n_heads, D)
    a, b = tf[..., : D // 2], tf[..., D // 2 :]
    c, s_ = c[:, None, :], s_[:, None, :]
    return torch.cat([a * c - b * s_, b * c + a * s_], -1).reshape(T, n_heads * D).to(t.dtype)


# ---------------------------------------------------------------------------- SwiGLU
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        T, I2 = gu.shape
        out = torch.empty(T, I2 // 2, dtype=gu.dtype, device=gu.device)
        rc = _lib.fn("vb_swiglu_fwd")(gu.data_ptr(), out.data_ptr(), T, I2 // 2, _lib.stream())
        _lib.check(rc, "vb_swiglu_fwd")
        ctx.save_for_backward(gu)
        return out

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        T, I2 = gu.shape
        dgu = torch.empty_like(gu)
        rc = _lib.fn("vb_swiglu_bwd")(gu.data_ptr(), dout.contiguous().data_ptr(), dgu.data_ptr(), T, I2 // 2,
                                      _lib.stream())
        _lib.check(rc, "vb_swiglu_bwd")
        return dgu


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up = [gate | up]`` along the last dim."""
    if gate_up.is_cuda:
        shape = gate_up.shape
        out = _SwiGLUFn.apply(gate_up.reshape(-1, shape[-1]).contiguous())
        return out.reshape(*shape[:-1], shape[-1] // 2)
    g, u = gate_up.chunk(2, dim=-1)
    return F.silu(g) * u


# ------------------------------------------------------------------------- Embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight):
        T = ids.numel()
        H = weight.shape[1]
        out = torch.empty(T, H, dtype=weight.dtype, device=weight.device)
        rc = _lib.fn("vb_embedding_fwd")(ids.data_ptr(), weight.data_ptr(), out.data_ptr(), T, H, _lib.stream())
        _lib.check(rc, "vb_embedding_fwd")
        ctx.save_for_backward(ids, weight)
        return out.reshape(*ids.shape, H)

    @staticmethod
    def backward(ctx, dy):
        ids, weight = ctx.saved_tensors
        T = ids.numel()
        H = weight.shape[1]
        main_grad = getattr(weight, "main_grad", None)
        buf = main_grad if main_grad is not None else torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        rc = _lib.fn("vb_embedding_bwd")(ids.data_ptr(), dy.reshape(T, H).contiguous().data_ptr(), buf.data_ptr(), T, H,
                                         _lib.stream())
        _lib.check(rc, "vb_embedding_bwd")
        return None, (None if main_grad is not None else buf.to(weight.dtype))


def embedding(ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    if weight.is_cuda:
        return _EmbeddingFn.apply(ids.contiguous(), weight)
    return F.embedding(ids, weight)
