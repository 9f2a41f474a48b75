"""Attention entry points.

* :func:`attention_varlen` — causal GQA attention over packed (remove-padding) sequences for
  training and prefill. On CUDA forward and backward are this package's tcgen05 kernels (head_dim 128);
  other head dims fall back to the ``flash_attn`` library (the reference uses it for everything through HF
  ``attn_implementation=flash_attention_2``, verl/workers/fsdp_workers.py:331). CPU: per-sequence SDPA loop.
* :func:`paged_decode_attention` / :func:`kv_cache_write` — the hand-written paged-KV decode
  path of the native rollout engine.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib

_flash = None


def _flash_varlen():
    global _flash
    if _flash is None:
        from flash_attn import flash_attn_varlen_func  # library kernel

        _flash = flash_attn_varlen_func
    return _flash


def flash_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int,
              causal: bool, scale: float, need_lse: bool = True, cu_seqlens_k: torch.Tensor | None = None):
    """tcgen05 forward. q [T,Hq,128], k/v [Tk,Hk,128] bf16 with unit inner strides (views of a fused qkv buffer are
    fine). ``cu_seqlens_k``: key-side boundaries when the keys are a longer stream than the queries (prefill on top
    of cached context; causal then aligns the queries with the end of the keys). ``max_seqlen`` is the longest
    query sequence. Returns (out [T,Hq,128] bf16, lse [Hq,T] fp32 or None)."""
    T, Hq, D = q.shape
    Hk = k.shape[1]
    for t in (q, k, v):
        if t.stride(2) != 1 or t.stride(1) != D or t.dtype != torch.bfloat16:
            raise ValueError("flash_fwd expects bf16 [T, H, 128] tensors with contiguous heads")
    out = torch.empty((T, Hq, D), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((Hq, T), dtype=torch.float32, device=q.device) if need_lse else None
    rc = _lib.fn("vb_flash_fwd")(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0), v.stride(0),
                                 cu_seqlens.data_ptr(), _lib.ptr(cu_seqlens_k), cu_seqlens.numel() - 1, T, k.shape[0],
                                 int(max_seqlen), Hq, Hk, float(scale),
                                 int(causal), out.data_ptr(), out.stride(0), _lib.ptr(lse),
                                 _lib.status_word(q.device).data_ptr(), _lib.stream())
    _lib.check(rc, "vb_flash_fwd")
    return out, lse


def flash_bwd(q, k, v, out, lse, dout, cu_seqlens, max_seqlen: int, causal: bool, scale: float):
    """tcgen05 backward: (dq [T,Hq,128], dk, dv [T,Hk,128]) from the forward's ``out`` and ``lse`` [Hq,T]."""
    T, Hq, D = q.shape
    Hk = k.shape[1]
    dout = dout if (dout.stride(2) == 1 and dout.stride(1) == D) else dout.contiguous()
    delta = torch.empty((Hq, T), dtype=torch.float32, device=q.device)
    dq = torch.empty((T, Hq, D), dtype=torch.bfloat16, device=q.device)
    dk = torch.empty((T, Hk, D), dtype=torch.bfloat16, device=q.device)
    dv = torch.empty_like(dk)
    st, stream = _lib.status_word(q.device).data_ptr(), _lib.stream()
    B = cu_seqlens.numel() - 1
    rc = _lib.fn("vb_flash_bwd_delta")(out.data_ptr(), dout.data_ptr(), out.stride(0), dout.stride(0), delta.data_ptr(), T, Hq, stream)
    _lib.check(rc, "vb_flash_bwd_delta")
    common = (q.data_ptr(), k.data_ptr(), v.data_ptr(), dout.data_ptr(), q.stride(0), k.stride(0), v.stride(0), dout.stride(0),
              cu_seqlens.data_ptr(), B, T, int(max_seqlen), Hq, Hk, float(scale), int(causal), lse.data_ptr(), delta.data_ptr())
    rc = _lib.fn("vb_flash_bwd_dq")(*common, dq.data_ptr(), dq.stride(0), st, stream)
    _lib.check(rc, "vb_flash_bwd_dq")
    rc = _lib.fn("vb_flash_bwd_dkv")(*common, dk.data_ptr(), dv.data_ptr(), dk.stride(0), st, stream)
    _lib.check(rc, "vb_flash_bwd_dkv")
    return dq, dk, dv


class _FlashVarlenFn(torch.autograd.Function):
    """Own forward and backward kernels (head_dim 128)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlen, causal, scale):
        out, lse = flash_fwd(q, k, v, cu_seqlens, max_seqlen, causal, scale)
        ctx.save_for_backward(q, k, v, out, lse, cu_seqlens)
        ctx.max_seqlen, ctx.causal, ctx.scale = max_seqlen, causal, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, cu = ctx.saved_tensors
        if _BWD_IMPL == "library":
            from flash_attn.flash_attn_interface import _flash_attn_varlen_backward  # library kernel

            qc, kc, vc = q.contiguous(), k.contiguous(), v.contiguous()
            dq, dk, dv = torch.empty_like(qc), torch.empty_like(kc), torch.empty_like(vc)
            _flash_attn_varlen_backward(dout.contiguous(), qc, kc, vc, out, lse, dq, dk, dv, cu, cu, ctx.max_seqlen,
                                        ctx.max_seqlen, 0.0, ctx.scale, ctx.causal, -1, -1, 0.0, None, False, None)
            return dq, dk, dv, None, None, None, None
        dq, dk, dv = flash_bwd(q, k, v, out, lse, dout, cu, ctx.max_seqlen, ctx.causal, ctx.scale)
        return dq, dk, dv, None, None, None, None


# "native" (default) or "library": which backward the autograd wrapper uses (the library one is kept for comparisons)
_BWD_IMPL = __import__("os").environ.get("VERL_B200_ATTN_BWD", "native")


def _native_fwd_ok(q, k, v) -> bool:
    D = q.shape[-1]
    return (q.dtype == torch.bfloat16 and D == 128 and q.shape[1] % k.shape[1] == 0
            and all(t.stride(2) == 1 and t.stride(1) == D and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0 for t in (q, k, v)))


def attention_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int,
                     causal: bool = True, softmax_scale: float | None = None, impl: str = "auto") -> torch.Tensor:
    """q [T,Hq,D], k/v [T,Hk,D] packed; cu_seqlens int32 [B+1]. Returns [T,Hq,D].
    ``impl``: "native" forces the tcgen05 forward, "library" the flash_attn kernels, "auto" picks native when it applies."""
    D = q.shape[-1]
    scale = softmax_scale if softmax_scale is not None else D ** -0.5
    if q.is_cuda:
        native = impl != "library" and _native_fwd_ok(q, k, v)
        if impl == "native" and not native:
            raise ValueError("native attention forward needs bf16, head_dim 128 and contiguous heads")
        if native:
            if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
                return _FlashVarlenFn.apply(q, k, v, cu_seqlens, int(max_seqlen), bool(causal), float(scale))
            return flash_fwd(q, k, v, cu_seqlens, int(max_seqlen), bool(causal), float(scale), need_lse=False)[0]
        return _flash_varlen()(q, k, v, cu_seqlens, cu_seqlens, max_seqlen, max_seqlen, softmax_scale=scale,
                               causal=causal)
    out = torch.empty_like(q)
    G = q.shape[1] // k.shape[1]
    bounds = cu_seqlens.tolist()
    for s, e in zip(bounds[:-1], bounds[1:]):
        qs = q[s:e].transpose(0, 1).unsqueeze(0)
        ks = k[s:e].repeat_interleave(G, dim=1).transpose(0, 1).unsqueeze(0)
        vs = v[s:e].repeat_interleave(G, dim=1).transpose(0, 1).unsqueeze(0)
        o = F.scaled_dot_product_attention(qs, ks, vs, is_causal=causal, scale=scale)
        out[s:e] = o.squeeze(0).transpose(0, 1)
    return out


def kv_cache_write(k: torch.Tensor, v: torch.Tensor, slots: torch.Tensor, k_cache: torch.Tensor,
                   v_cache: torch.Tensor) -> None:
    """Scatter new keys/values [T,Hk,D] into the paged caches [NB,Hk,BS,D] at flat ``slots`` (int64, <0 skips)."""
    T, Hk, D = k.shape
    BS = k_cache.shape[2]
    if k.is_cuda:
        rc = _lib.fn("vb_kv_cache_write")(k.data_ptr(), v.data_ptr(), k.stride(0), v.stride(0), slots.data_ptr(),
                                          k_cache.data_ptr(), v_cache.data_ptr(), T, Hk, D, BS, _lib.stream())
        _lib.check(rc, "vb_kv_cache_write")
        return
    ok = slots >= 0
    blk, off = slots[ok] // BS, slots[ok] % BS
    k_cache[blk, :, off] = k[ok]
    v_cache[blk, :, off] = v[ok]


def decode_workspace(B: int, Hq: int, Hk: int, D: int, max_seq_len: int, device) -> tuple[int, torch.Tensor | None]:
    """Split count and fp32 scratch for :func:`paged_decode_attention` at these sizes."""
    if torch.device(device).type != "cuda":
        return 1, None
    splits = _lib.fn("vb_decode_num_splits")(B, Hk, max_seq_len)
    work = torch.empty(B * Hq * splits * (D + 2), dtype=torch.float32, device=device) if splits > 1 else None
    return splits, work


def paged_decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                           seq_lens: torch.Tensor, scale: float | None = None, num_splits: int = 1,
                           work: torch.Tensor | None = None, out: torch.Tensor | None = None,
                           impl: str = "auto") -> torch.Tensor:
    """One query token per sequence. q [B,Hq,D]; caches [NB,Hk,BS,D]; block_table int32 [B,max_blocks];
    seq_lens int32 [B] (including the current token, already written to the cache).

    ``impl``: "tc" = tcgen05 kernel (head_dim 128, <= 16 query heads per KV head, block size a power of two in
    8..128), "simt" = CUDA-core kernel, "auto" = "tc" wherever it applies."""
    B, Hq, D = q.shape
    Hk, BS = k_cache.shape[1], k_cache.shape[2]
    scale = scale if scale is not None else D ** -0.5
    if out is None:
        out = torch.empty_like(q)
    if q.is_cuda:
        if num_splits > 1 and work is None:
            work = torch.empty(B * Hq * num_splits * (D + 2), dtype=torch.float32, device=q.device)
        tc_ok = bool(_lib.fn("vb_paged_decode_tc_supported")(Hq, Hk, D, BS)) and k_cache.is_contiguous() and v_cache.is_contiguous()
        if impl == "tc" and not tc_ok:
            raise ValueError(f"tensor-core decode does not support Hq={Hq} Hk={Hk} D={D} block_size={BS}")
        if tc_ok and impl != "simt":
            rc = _lib.fn("vb_paged_decode_tc")(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
                                               k_cache.shape[0], block_table.data_ptr(), block_table.stride(0),
                                               seq_lens.data_ptr(), B, Hq, Hk, BS, scale, num_splits, out.data_ptr(),
                                               out.stride(0), _lib.ptr(work), _lib.status_word(q.device).data_ptr(),
                                               _lib.stream())
            _lib.check(rc, "vb_paged_decode_tc")
            return out
        rc = _lib.fn("vb_paged_decode")(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
                                        block_table.data_ptr(), block_table.stride(0), seq_lens.data_ptr(), B, Hq, Hk,
                                        D, BS, scale, num_splits, out.data_ptr(), out.stride(0), _lib.ptr(work),
                                        _lib.stream())
        _lib.check(rc, "vb_paged_decode")
        return out
    G = Hq // Hk
    for b in range(B):
        L = int(seq_lens[b])
        nb = (L + BS - 1) // BS
        blocks = block_table[b, :nb].long()
        kk = k_cache[blocks].permute(1, 0, 2, 3).reshape(Hk, -1, D)[:, :L].float()
        vv = v_cache[blocks].permute(1, 0, 2, 3).reshape(Hk, -1, D)[:, :L].float()
        qq = q[b].float().reshape(Hk, G, D)
        s = torch.einsum("hgd,hld->hgl", qq, kk) * scale
        out[b] = torch.einsum("hgl,hld->hgd", torch.softmax(s, -1), vv).reshape(Hq, D).to(q.dtype)
    return out
