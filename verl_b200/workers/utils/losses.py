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


# ---------------------------------------------------------------------------------------------------------------
# Loss functions of the TensorDict batch interface (``engine.forward_backward_batch``): called as
# ``fn(model_output=..., data=micro_batch, dp_group=...)`` after ``functools.partial(fn, config)``; the engine has put
# ``dp_size``, ``batch_num_tokens`` and ``global_batch_size`` (sums over the data-parallel group) into ``data``.
# Semantics of verl/workers/utils/losses.py:27-214.
def _nt(data, key, default=None):
    from ...utils import tensordict_utils as tu

    return tu.get(data, key, default)


def slice_response_from_unpad_output(tensor: torch.Tensor, data) -> torch.Tensor:
    """Per-token model output aligned with the packed ``input_ids`` -> padded ``[bsz, max_response_len]`` tensor of
    the response part, shifted left by one (output ``t`` scores token ``t + 1``)."""
    values = tensor.values() if tensor.is_nested else tensor
    prompts, responses, attn = data["prompts"], data["responses"], data["attention_mask"]
    if prompts.is_nested:
        p_len, r_len = prompts.offsets().diff(), responses.offsets().diff()
        max_r = int(r_len.max().item())
    else:
        p_len = attn[:, : prompts.shape[1]].sum(1)
        r_len = attn[:, prompts.shape[1]:].sum(1)
        max_r = responses.shape[1]
    ends = (p_len + r_len).cumsum(0)
    assert int(ends[-1]) == values.shape[0], (int(ends[-1]), values.shape)
    rows = []
    for rl, e in zip(r_len.tolist(), ends.tolist()):
        rows.append(torch.nn.functional.pad(values[e - rl - 1 : e - 1], (0, max_r - rl)))
    return torch.stack(rows, 0)


def sft_loss_on_batch(config, model_output, data, dp_group=None):
    lp = model_output["log_probs"]
    if lp.is_nested:
        mask = torch.roll(data["loss_mask"].values().to(lp.values().device), -1, 0).to(lp.values().dtype)
        total = (lp.values() * mask).sum()
    else:
        total = (lp * data["response_mask"].to(lp.dtype)).sum()
    loss = -total / max(float(_nt(data, "batch_num_tokens", 1.0)), 1.0) * int(_nt(data, "dp_size", 1))
    return loss, {}


def ppo_loss_on_batch(config, model_output, data, dp_group=None):
    lp = slice_response_from_unpad_output(model_output["log_probs"], data)
    ent = model_output.get("entropy")
    if ent is not None:
        ent = slice_response_from_unpad_output(ent, data)
    info = {"dp_size": int(_nt(data, "dp_size", 1)), "batch_num_tokens": _nt(data, "batch_num_tokens"),
            "global_batch_size": _nt(data, "global_batch_size"), "loss_scale_factor": _cfg(config, "loss_scale_factor", None)}
    if isinstance(config, dict):
        config["global_batch_info"] = info
    else:
        object.__setattr__(config, "global_batch_info", info)
    dev = lp.device
    fields = {k: data[k].to(dev) for k in ("response_mask", "old_log_probs", "advantages", "ref_log_prob", "rollout_is_weights")
              if k in data.keys()}
    loss, metrics = ppo_loss(config, lp, ent, fields)
    return loss, {k: float(v) for k, v in metrics.items()}


def value_loss_on_batch(config, model_output, data, dp_group=None):
    vp = slice_response_from_unpad_output(model_output["values"], data)
    dev = vp.device
    fields = {k: data[k].to(dev) for k in ("values", "returns", "response_mask")}
    loss, metrics = value_loss(config, vp, fields)
    return loss, {k: float(v) for k, v in metrics.items()}
