"""Loss functions on engine outputs (verl/workers/utils/losses.py:1-214): each takes per-token model outputs
plus the batch fields and returns (loss, metrics)."""

from __future__ import annotations

import torch

from ...trainer.ppo import core_algos


def _cfg(c, k, d=None):
    if c is None:
        return d
    v = c.get(k, d) if hasattr(c, "get") else getattr(c, k, d)
    return d if v is None else v


def sft_loss(log_prob: torch.Tensor, loss_mask: torch.Tensor, global_tokens: float | None = None, dp_size: int = 1):
    """Mean negative log-likelihood over the masked tokens. With ``global_tokens`` (sum of the mask over all
    data-parallel ranks and micro-batches) the per-micro-batch losses add up to the global token mean after the
    gradient reduction, which sums over ranks."""
    mask = loss_mask.to(log_prob.dtype)
    if global_tokens is None:
        loss = -(log_prob * mask).sum() / mask.sum().clamp(min=1.0)
    else:
        loss = -(log_prob * mask).sum() / max(float(global_tokens), 1.0) * dp_size
    return loss, {"sft/loss": loss.detach()}


def ppo_loss(config, log_prob, entropy, data: dict, loss_scale: float = 1.0):
    """Policy loss (registry lookup by ``policy_loss.loss_mode``) + entropy bonus + KL loss."""
    mask = data["response_mask"]
    mode = _cfg(_cfg(config, "policy_loss", {}), "loss_mode", "vanilla")
    agg = _cfg(config, "loss_agg_mode", "token-mean")
    fn = core_algos.get_policy_loss_fn(mode)
    pg_loss, pg_metrics = fn(old_log_prob=data["old_log_probs"], log_prob=log_prob, advantages=data["advantages"],
                             response_mask=mask, loss_agg_mode=agg, config=config,
                             rollout_is_weights=data.get("rollout_is_weights"))
    metrics = {f"actor/{k}" if not k.startswith("actor/") else k: v for k, v in (pg_metrics or {}).items()}
    loss = pg_loss
    coef = float(_cfg(config, "entropy_coeff", 0.0) or 0.0)
    if coef != 0.0 and entropy is not None:
        ent = core_algos.agg_loss(entropy, mask, agg)
        loss = loss - coef * ent
        metrics["actor/entropy"] = ent.detach()
    if _cfg(config, "use_kl_loss", False) and "ref_log_prob" in data:
        kld = core_algos.kl_penalty(log_prob, data["ref_log_prob"], _cfg(config, "kl_loss_type", "low_var_kl"))
        kl = core_algos.agg_loss(kld, mask, agg)
        loss = loss + float(_cfg(config, "kl_loss_coef", 0.001)) * kl
        metrics["actor/kl_loss"] = kl.detach()
    metrics["actor/pg_loss"] = pg_loss.detach()
    return loss * loss_scale, metrics


def value_loss(config, vpreds, data: dict, loss_scale: float = 1.0):
    vf_loss, clipfrac = core_algos.compute_value_loss(
        vpreds=vpreds, values=data["values"], returns=data["returns"], response_mask=data["response_mask"],
        cliprange_value=float(_cfg(config, "cliprange_value", 0.5)), loss_agg_mode=_cfg(config, "loss_agg_mode", "token-mean"))
    return vf_loss * loss_scale, {"critic/vf_loss": vf_loss.detach(), "critic/vf_clipfrac": clipfrac.detach()}
