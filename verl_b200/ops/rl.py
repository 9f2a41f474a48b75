"""RL math on the GPU: fused PPO token loss, GAE scan, GRPO advantages, sampler, fused AdamW.

Each function has the same semantics as the torch formulation in
:mod:`verl_b200.trainer.ppo.core_algos` (which follows verl/trainer/ppo/core_algos.py); the
CUDA path does the whole computation in one or two launches.
"""

from __future__ import annotations

import torch

from . import _lib

KL_TYPES = {"kl": 0, "k1": 0, "abs": 1, "mse": 2, "k2": 2, "low_var_kl": 3, "k3": 3}
PPO_METRIC_NAMES = ("pg_loss", "pg_clipfrac", "ppo_kl", "pg_clipfrac_lower", "kl_loss", "entropy", "num_tokens")


class _PPOLossFn(torch.autograd.Function):
    """Token-mean PPO loss: sum_t mask * (pg - c_ent * entropy + c_kl * kl) * inv_denom.

    Gradient and the seven metric sums are produced by the same pass; ``metrics`` is a detached
    fp32[7] tensor of *sums* over masked tokens (see ``PPO_METRIC_NAMES``)."""

    @staticmethod
    def forward(ctx, logp, entropy, old_logp, adv, mask, ref_logp, is_weight, clip_low, clip_high, clip_c, kl_coef,
                kl_type, entropy_coeff, inv_denom):
        n = logp.numel()
        dev = logp.device
        d_logp = torch.empty(n, dtype=torch.float32, device=dev)
        d_ent = torch.empty(n, dtype=torch.float32, device=dev) if entropy is not None else None
        metrics = torch.zeros(8, dtype=torch.float32, device=dev)

        def c(t):
            return None if t is None else t.reshape(-1).float().contiguous()

        tensors = [c(logp), c(old_logp), c(adv), c(mask), c(ref_logp), c(entropy), c(is_weight)]
        rc = _lib.fn("vb_ppo_loss")(*[_lib.ptr(t) for t in tensors], d_logp.data_ptr(), _lib.ptr(d_ent),
                                    metrics.data_ptr(), n, clip_low, clip_high, clip_c, kl_coef, kl_type,
                                    entropy_coeff, inv_denom, _lib.stream())
        _lib.check(rc, "vb_ppo_loss")
        ctx.save_for_backward(d_logp, d_ent)
        ctx.shape = logp.shape
        ctx.has_ent = entropy is not None
        loss = (metrics[0] - entropy_coeff * metrics[5] + kl_coef * metrics[4]) * inv_denom
        ctx.mark_non_differentiable(metrics)
        return loss, metrics

    @staticmethod
    def backward(ctx, g_loss, _g_metrics):
        d_logp, d_ent = ctx.saved_tensors
        gl = (d_logp * g_loss).reshape(ctx.shape)
        ge = (d_ent * g_loss).reshape(ctx.shape) if ctx.has_ent else None
        return (gl, ge) + (None,) * 12


def ppo_loss_fused(logp, old_logp, adv, mask, *, entropy=None, ref_logp=None, is_weight=None, clip_low=0.2,
                   clip_high=0.2, clip_c=3.0, kl_coef=0.0, kl_type="low_var_kl", entropy_coeff=0.0,
                   denom: float | None = None):
    """Returns ``(loss, metric_sums)``. ``denom`` is the token count the loss is normalised by
    (token-mean; pass the global count for DP-consistent scaling); default = local mask sum."""
    if denom is None:
        denom = float(mask.sum().clamp(min=1.0))
    use_kl = ref_logp is not None and kl_coef != 0.0
    return _PPOLossFn.apply(logp, entropy if entropy_coeff != 0.0 or entropy is not None else None, old_logp, adv,
                            mask, ref_logp if use_kl else None, is_weight, float(clip_low), float(clip_high),
                            float(clip_c), float(kl_coef if use_kl else 0.0), KL_TYPES[kl_type], float(entropy_coeff),
                            1.0 / float(denom))


def gae(rewards: torch.Tensor, values: torch.Tensor, mask: torch.Tensor, gamma: float, lam: float):
    """Reverse-scan GAE on [B,T] fp32 tensors -> (advantages, returns), before whitening."""
    B, T = rewards.shape
    r, v, m = rewards.float().contiguous(), values.float().contiguous(), mask.float().contiguous()
    adv, ret = torch.empty_like(r), torch.empty_like(r)
    rc = _lib.fn("vb_gae")(r.data_ptr(), v.data_ptr(), m.data_ptr(), adv.data_ptr(), ret.data_ptr(), B, T,
                           float(gamma), float(lam), _lib.stream())
    _lib.check(rc, "vb_gae")
    return adv, ret


def grpo_advantage(scores: torch.Tensor, group_ids: torch.Tensor, mask: torch.Tensor, num_groups: int,
                   eps: float = 1e-6, norm_by_std: bool = True) -> torch.Tensor:
    """scores [B] fp32, group_ids [B] int32 in [0,num_groups), mask [B,T] -> advantages [B,T]."""
    B, T = mask.shape
    s, g, m = scores.float().contiguous(), group_ids.int().contiguous(), mask.float().contiguous()
    adv = torch.empty_like(m)
    work = torch.empty(3 * num_groups, dtype=torch.float32, device=m.device)
    rc = _lib.fn("vb_grpo_adv")(s.data_ptr(), g.data_ptr(), m.data_ptr(), adv.data_ptr(), work.data_ptr(), B, T,
                                num_groups, float(eps), int(norm_by_std), _lib.stream())
    _lib.check(rc, "vb_grpo_adv")
    return adv


def sample(logits: torch.Tensor, *, temperature: torch.Tensor | None = None, top_k: torch.Tensor | None = None,
           top_p: torch.Tensor | None = None, seed: int = 0, step: torch.Tensor | None = None,
           out_tokens: torch.Tensor | None = None, out_logprobs: torch.Tensor | None = None):
    """Sample one token per row of ``logits`` [B,V] (fp32 or bf16). Per-row device arrays:
    temperature fp32 (<=0 -> greedy), top_k int32 (<=0 off), top_p fp32 (>=1 off). ``step`` is an int64
    device counter mixed into the Philox stream. Returns (tokens int64 [B], logprobs fp32 [B])."""
    B, V = logits.shape
    if out_tokens is None:
        out_tokens = torch.empty(B, dtype=torch.long, device=logits.device)
    if out_logprobs is None:
        out_logprobs = torch.empty(B, dtype=torch.float32, device=logits.device)
    if not logits.is_cuda:
        lg = logits.float()
        t = temperature if temperature is not None else torch.ones(B)
        greedy = t <= 1e-6
        lg = lg / torch.where(greedy, torch.ones_like(t), t)[:, None]
        lp = torch.log_softmax(lg, -1)
        gen = torch.Generator().manual_seed(int(seed) + (int(step.item()) if step is not None else 0))
        tok = torch.multinomial(lp.exp(), 1, generator=gen)[:, 0]
        tok = torch.where(greedy, lg.argmax(-1), tok)
        out_tokens.copy_(tok)
        out_logprobs.copy_(lp.gather(1, tok[:, None])[:, 0])
        return out_tokens, out_logprobs
    dtype = 0 if logits.dtype == torch.float32 else 1
    rc = _lib.fn("vb_sample")(logits.data_ptr(), dtype, logits.stride(0), B, V, _lib.ptr(temperature), _lib.ptr(top_k),
                              _lib.ptr(top_p), int(seed), _lib.ptr(step), out_tokens.data_ptr(),
                              out_logprobs.data_ptr(), _lib.stream())
    _lib.check(rc, "vb_sample")
    return out_tokens, out_logprobs


def decode_advance(tok, lp, ids, pos, slots, lens, bt, block_size: int, limit, alive, flags, eos: int, ring_tok, ring_lp,
                   bpos, sampler_step=None) -> None:
    """Last op of a decode step: store the sampled tokens / log-probs in row ``bpos`` of the burst ring and turn them into
    the next step's inputs in place (``ids, pos, slots, lens``); rows that sample ``eos`` (unless ``flags`` bit 0) or
    reach ``limit`` tokens stop advancing (``alive`` 0, slot -1). Also advances ``bpos`` and the sampler's step counter."""
    B = tok.numel()
    kmax = ring_tok.shape[0]
    if tok.is_cuda:
        rc = _lib.fn("vb_decode_advance")(tok.data_ptr(), lp.data_ptr(), ids.data_ptr(), pos.data_ptr(), slots.data_ptr(),
                                          lens.data_ptr(), bt.data_ptr(), bt.shape[1], int(block_size), limit.data_ptr(),
                                          alive.data_ptr(), flags.data_ptr(), int(eos), ring_tok.data_ptr(),
                                          ring_lp.data_ptr(), bpos.data_ptr(), _lib.ptr(sampler_step), B, kmax, _lib.stream())
        _lib.check(rc, "vb_decode_advance")
        return
    s = int(bpos.item())
    a = alive.bool()
    if 0 <= s < kmax:
        ring_tok[s] = torch.where(a, tok, torch.full_like(tok, -1))
        ring_lp[s] = torch.where(a, lp, torch.zeros_like(lp))
    ti = lens.long() - 1  # index of the token just processed (the RoPE position may be offset from it)
    done = a & ((((flags & 1) == 0) & (tok == eos)) | (ti + 2 >= limit.long()))
    go = a & ~done
    p = ti + 1
    blk = torch.div(p, block_size, rounding_mode="floor").clamp(max=bt.shape[1] - 1)
    new_slot = bt.long().gather(1, blk[:, None])[:, 0] * block_size + p % block_size
    ids.copy_(torch.where(go, tok, ids))
    pos.copy_(torch.where(go, pos + 1, pos))
    lens.copy_(torch.where(go, lens + 1, lens))
    slots.copy_(torch.where(go, new_slot, torch.where(done, torch.full_like(slots, -1), slots)))
    alive.copy_(torch.where(done, torch.zeros_like(alive), alive))
    bpos.add_(1)
    if sampler_step is not None:
        sampler_step.add_(1)


# ------------------------------------------------------------------------- optimizer
def adamw_step(p32, grad, m, v, p16, *, lr, betas, eps, weight_decay, step, scale=None, skip=None):
    """Fused AdamW on a flat fp32 master shard; also refreshes the bf16 working copy ``p16``.
    ``scale`` (fp32[1], device) multiplies the gradient; ``skip`` (int32[1], device) != 0 is a no-op."""
    n = p32.numel()
    rc = _lib.fn("vb_adamw")(p32.data_ptr(), grad.data_ptr(), int(grad.dtype == torch.bfloat16), m.data_ptr(),
                             v.data_ptr(), _lib.ptr(p16), n, float(lr), float(betas[0]), float(betas[1]), float(eps),
                             float(weight_decay), int(step), _lib.ptr(scale), _lib.ptr(skip), _lib.stream())
    _lib.check(rc, "vb_adamw")


def sumsq_into(x: torch.Tensor, out: torch.Tensor) -> None:
    """out[0] += sum(x^2) for a flat fp32/bf16 tensor."""
    rc = _lib.fn("vb_sumsq")(x.data_ptr(), int(x.dtype == torch.bfloat16), x.numel(), out.data_ptr(), _lib.stream())
    _lib.check(rc, "vb_sumsq")


def clip_coef(sumsq: torch.Tensor, max_norm: float, extra_scale: float, scale_out: torch.Tensor,
              skip_out: torch.Tensor, norm_out: torch.Tensor) -> None:
    rc = _lib.fn("vb_clip_coef")(sumsq.data_ptr(), float(max_norm), float(extra_scale), scale_out.data_ptr(),
                                 skip_out.data_ptr(), norm_out.data_ptr(), _lib.stream())
    _lib.check(rc, "vb_clip_coef")
