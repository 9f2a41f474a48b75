"""Rollout correction: truncated importance weights, divergence-based rejection masks and
off-policy diagnostics between the training policy and the rollout policy.

Same entry points, option names and metric keys as verl/trainer/ppo/rollout_corr_helper.py
(rejection :156-330, IS weights :481-560, combined :716-830, off-policy metrics :834-940,
batch glue :943-1074). Everything is in log space with ``SAFETY_BOUND = 20``. Option handling is
table-driven: ``<level>_<estimator>`` = (how token statistics are pooled) x (k1 | k2 | k3).
"""

from __future__ import annotations

import math
from typing import Any, Optional

import torch

from ...protocol import DataProto
from ...utils import torch_functional as F_

SAFETY_BOUND = 20.0

TOKEN_LEVEL_ROLLOUT_RS_OPTIONS = {"token_k1", "token_k2", "token_k3"}
SUPPORTED_ROLLOUT_RS_OPTIONS = TOKEN_LEVEL_ROLLOUT_RS_OPTIONS | {
    "seq_sum_k1", "seq_sum_k2", "seq_sum_k3", "seq_mean_k1", "seq_mean_k2", "seq_mean_k3", "seq_max_k2", "seq_max_k3",
}


def _parse_rollout_rs_thresholds(options: list[str], threshold_spec) -> dict[str, dict[str, Optional[float]]]:
    """k1 options take "lower_upper" (or "upper", lower = 1/upper); k2/k3 take a single upper bound."""
    if threshold_spec is None:
        raise ValueError("rollout_rs_threshold must be provided for rejection sampling.")
    if isinstance(threshold_spec, (int, float)):
        specs = [str(threshold_spec)]
    elif isinstance(threshold_spec, str):
        specs = [s.strip() for s in threshold_spec.split(",") if s.strip()]
    else:
        raise TypeError("rollout_rs_threshold must be a string or numeric value specifying per-option thresholds.")
    if not specs:
        raise ValueError("rollout_rs_threshold must contain at least one threshold value.")
    if len(specs) not in (1, len(options)):
        raise ValueError(f"rollout_rs_threshold expects either one threshold shared by all options or exactly "
                         f"{len(options)} thresholds to match the provided rollout_rs options.")
    if len(specs) == 1:
        specs = specs * len(options)
    out = {}
    for opt, spec in zip(options, specs):
        try:
            if opt.endswith("k1"):
                lo_s, hi_s = spec.split("_", 1) if "_" in spec else (None, spec)
                hi = float(hi_s)
                lo = float(lo_s) if lo_s is not None else 1.0 / hi
                if lo <= 0 or hi <= 0:
                    raise ValueError(f"Thresholds for option '{opt}' must be positive, got {spec}.")
                out[opt] = {"lower": lo, "upper": hi}
            else:
                if "_" in spec:
                    raise ValueError(f"rollout_rs_threshold for option '{opt}' must provide a single upper bound "
                                     f"without '_'. Received '{spec}'.")
                hi = float(spec)
                if hi <= 0:
                    raise ValueError(f"Threshold for option '{opt}' must be positive, got {spec}.")
                out[opt] = {"lower": None, "upper": hi}
        except ValueError as exc:
            if "must" in str(exc):
                raise
            raise ValueError(f"Invalid numeric threshold '{spec}' for option '{opt}'.") from exc
    return out


def _seq_max(values: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    mx = values.masked_fill(~mask.bool(), float("-inf")).max(dim=-1).values
    return torch.where(torch.isinf(mx) & (mx < 0), torch.zeros_like(mx), mx)


_POOL = {
    "seq_sum": lambda v, m: F_.masked_sum(v, m, axis=-1),
    "seq_mean": lambda v, m: F_.masked_mean(v, m, axis=-1),
    "seq_max": _seq_max,
}


def compute_rs_metrics(option_name: str, rs_statistic: torch.Tensor, response_mask: torch.Tensor,
                       seq_valid_mask: torch.Tensor, *, level: str, per_sequence_values: Optional[torch.Tensor],
                       rollout_rs_threshold: float, rollout_rs_threshold_lower: float,
                       apply_lower_threshold: bool) -> dict[str, float]:
    if not response_mask.any():
        raise ValueError("response_mask must contain at least one valid token (1).")
    m: dict[str, float] = {}
    pre = f"rollout_rs_{option_name}"
    mb = response_mask.bool()
    seq_vals = per_sequence_values if per_sequence_values is not None else F_.masked_mean(rs_statistic, response_mask, axis=-1)
    seq_vals = seq_vals.reshape(-1)[seq_valid_mask]
    hi, lo = rollout_rs_threshold, rollout_rs_threshold_lower
    m[f"{pre}_mean"] = F_.masked_mean(rs_statistic, response_mask).item()
    use_seq = level == "sequence" and seq_vals.numel() > 0
    if use_seq:
        m[f"{pre}_max"], m[f"{pre}_min"] = seq_vals.max().item(), seq_vals.min().item()
        m[f"{pre}_fraction_high"] = (seq_vals > hi).float().mean().item()
        m[f"{pre}_fraction_low"] = (seq_vals < lo).float().mean().item() if apply_lower_threshold else 0.0
    else:
        m[f"{pre}_max"] = rs_statistic.masked_fill(~mb, float("-inf")).max().item()
        m[f"{pre}_min"] = rs_statistic.masked_fill(~mb, float("inf")).min().item()
        m[f"{pre}_fraction_high"] = F_.masked_mean((rs_statistic > hi).float(), response_mask).item()
        m[f"{pre}_fraction_low"] = (F_.masked_mean((rs_statistic < lo).float(), response_mask).item()
                                    if apply_lower_threshold else 0.0)
    if response_mask.sum() > 1:
        c = rs_statistic.clamp(min=lo if apply_lower_threshold else 0.0, max=hi)
        var = F_.masked_mean(c.square(), response_mask) - F_.masked_mean(c, response_mask).square()
        m[f"{pre}_std"] = torch.sqrt(torch.clamp(var, min=0.0)).item()
    else:
        m[f"{pre}_std"] = 0.0
    if seq_vals.numel() > 0:
        m[f"{pre}_seq_mean"] = seq_vals.mean().item()
        m[f"{pre}_seq_std"] = seq_vals.std().item() if seq_vals.numel() > 1 else 0.0
        m[f"{pre}_seq_max"], m[f"{pre}_seq_min"] = seq_vals.max().item(), seq_vals.min().item()
        m[f"{pre}_seq_max_deviation"] = seq_vals.abs().max().item()
        m[f"{pre}_seq_fraction_high"] = (seq_vals > hi).float().mean().item()
        if apply_lower_threshold:
            m[f"{pre}_seq_fraction_low"] = (seq_vals < lo).float().mean().item()
    else:
        for k in ("mean", "std", "max", "min", "max_deviation", "fraction_high", "fraction_low"):
            m[f"{pre}_seq_{k}"] = 0.0
    return m


def compute_rollout_rejection_mask(log_ratio: torch.Tensor, response_mask: torch.Tensor, rollout_rs: str = "token_k1",
                                   rollout_rs_threshold=None) -> tuple[torch.Tensor, dict[str, float]]:
    """Zero the mask of tokens (token_*) or whole sequences (seq_*) whose divergence statistic is out of range.
    Several comma-separated options intersect."""
    if rollout_rs is None or not isinstance(rollout_rs, str):
        raise ValueError("rollout_rs must be a non-empty string (comma separated for multiple options).")
    if rollout_rs_threshold is None:
        raise ValueError("rollout_rs_threshold must be provided for rejection sampling.")
    if log_ratio.shape[0] == 0:
        return response_mask, {}
    opts = []
    for o in (x.strip() for x in rollout_rs.split(",")):
        if not o:
            continue
        if o not in SUPPORTED_ROLLOUT_RS_OPTIONS:
            raise ValueError(f"Invalid rollout_rs option: {o}. Must be one of {sorted(SUPPORTED_ROLLOUT_RS_OPTIONS)}.")
        if o not in opts:
            opts.append(o)
    if not opts:
        raise ValueError("rollout_rs must contain at least one valid option.")
    thr = _parse_rollout_rs_thresholds(opts, rollout_rs_threshold)
    lr = torch.clamp(log_ratio, min=-SAFETY_BOUND, max=SAFETY_BOUND)
    stats = {"k1": -lr, "k2": 0.5 * lr ** 2, "k3": torch.exp(lr) - 1.0 - lr}
    mask_b = response_mask.bool()
    seq_valid = response_mask.sum(dim=-1) > 0
    keep_all = torch.ones_like(response_mask, dtype=log_ratio.dtype)
    metrics: dict[str, float] = {}
    for opt in opts:
        level_name, est = opt.rsplit("_", 1)
        is_k1 = est == "k1"
        hi, lo = thr[opt]["upper"], thr[opt]["lower"]
        if is_k1:
            if lo is None or hi is None:
                raise ValueError(f"rollout_rs_threshold for option '{opt}' must specify both lower and upper bounds.")
            hi_cmp, lo_cmp = math.log(hi), math.log(lo)
        else:
            hi_cmp, lo_cmp = hi, 0.0
        tok = stats[est]
        if level_name == "token":
            stat, seq_stat, level = tok, None, "token"
        else:
            seq_stat = _POOL[level_name](tok, response_mask)
            stat, level = seq_stat.unsqueeze(-1).expand_as(response_mask), "sequence"
        keep = (stat <= hi_cmp) & ((stat >= lo_cmp) if is_k1 else torch.ones_like(stat, dtype=torch.bool))
        keep_f = keep.to(log_ratio.dtype)
        keep_all = keep_all * keep_f
        metrics.update(compute_rs_metrics(opt, stat, response_mask, seq_valid, level=level, per_sequence_values=seq_stat,
                                          rollout_rs_threshold=hi_cmp, rollout_rs_threshold_lower=lo_cmp,
                                          apply_lower_threshold=is_k1))
        seq_keep = (~((~keep) & mask_b)).all(dim=-1).to(log_ratio.dtype)
        sv = seq_valid.float()
        metrics[f"rollout_rs_{opt}_masked_fraction"] = F_.masked_mean(1 - keep_f, response_mask).item()
        metrics[f"rollout_rs_{opt}_seq_masked_fraction"] = (((1.0 - seq_keep) * sv).sum() / sv.sum()).item() if sv.sum() > 0 else 0.0
    metrics["rollout_rs_masked_fraction"] = F_.masked_mean(1 - keep_all, response_mask).item()
    kept = (keep_all > 0.5) & mask_b
    metrics["rollout_rs_seq_masked_fraction"] = (~kept & mask_b).any(dim=-1).float().mean().item()
    return (response_mask * keep_all).to(response_mask.dtype), metrics


def compute_is_metrics(rollout_is_weights: torch.Tensor, log_ratio_for_metrics: torch.Tensor, response_mask: torch.Tensor,
                       rollout_is: str, rollout_is_threshold: float) -> dict[str, float]:
    if not response_mask.any():
        raise ValueError("response_mask must contain at least one valid token (1).")
    m: dict[str, float] = {}
    w = rollout_is_weights
    hi, lo = rollout_is_threshold, 1.0 / rollout_is_threshold
    m["rollout_is_mean"] = F_.masked_mean(w, response_mask).item()
    if rollout_is == "sequence":
        lmax, lmin = log_ratio_for_metrics.max(), log_ratio_for_metrics.min()
        m["rollout_is_max"] = torch.exp(torch.clamp(lmax, max=SAFETY_BOUND)).item()
        m["rollout_is_min"] = torch.exp(lmin).item()
        m["rollout_is_ratio_fraction_high"] = (log_ratio_for_metrics > math.log(hi)).float().mean().item()
        m["rollout_is_ratio_fraction_low"] = (log_ratio_for_metrics < math.log(lo)).float().mean().item()
    else:
        mb = response_mask.bool()
        m["rollout_is_ratio_fraction_high"] = F_.masked_mean((w > hi).float(), response_mask).item()
        m["rollout_is_ratio_fraction_low"] = F_.masked_mean((w < lo).float(), response_mask).item()
        m["rollout_is_max"] = w.masked_fill(~mb, float("-inf")).max().item()
        m["rollout_is_min"] = w.masked_fill(~mb, float("inf")).min().item()
    wc = w.clamp(min=lo, max=hi)
    if response_mask.sum() > 1:
        var = F_.masked_mean(wc.square(), response_mask) - F_.masked_mean(wc, response_mask).square()
        m["rollout_is_std"] = torch.sqrt(torch.clamp(var, min=0.0)).item()
    else:
        m["rollout_is_std"] = 0.0
    wn = wc / (F_.masked_mean(wc, response_mask) + 1e-8)
    m["rollout_is_eff_sample_size"] = 1.0 / F_.masked_mean(wn.square(), response_mask).item()
    if w.dim() > 1:
        sm = F_.masked_mean(w, response_mask, axis=-1)
        m["rollout_is_seq_mean"] = sm.mean().item()
        m["rollout_is_seq_std"] = sm.std().item() if sm.numel() > 1 else 0.0
        m["rollout_is_seq_max"], m["rollout_is_seq_min"] = sm.max().item(), sm.min().item()
        m["rollout_is_seq_max_deviation"] = (sm - 1.0).abs().max().item()
        m["rollout_is_seq_fraction_high"] = (sm > hi).float().mean().item()
        m["rollout_is_seq_fraction_low"] = (sm < lo).float().mean().item()
    return m


def compute_rollout_correction_weights(log_ratio: torch.Tensor, response_mask: torch.Tensor, rollout_is: str = "token",
                                       rollout_is_threshold: float = 2.0,
                                       rollout_is_batch_normalize: bool = False) -> tuple[torch.Tensor, dict[str, float]]:
    """Truncated importance weights min(exp(log-ratio), threshold) at token or sequence level."""
    if rollout_is not in ("token", "sequence"):
        raise ValueError(f"Invalid rollout_is: {rollout_is}. Must be one of {{'token', 'sequence'}}.")
    if rollout_is_threshold <= 0:
        raise ValueError(f"rollout_is_threshold must be positive, got {rollout_is_threshold}.")
    if rollout_is == "token":
        lr_m = log_ratio
        w = torch.exp(torch.clamp(log_ratio, min=-SAFETY_BOUND, max=SAFETY_BOUND))
    else:
        lr_m = F_.masked_sum(log_ratio, response_mask, axis=-1).unsqueeze(-1)
        w = torch.exp(torch.clamp(lr_m, min=-SAFETY_BOUND, max=SAFETY_BOUND)).expand_as(log_ratio)
    w = w * response_mask
    metrics = compute_is_metrics(w, lr_m, response_mask, rollout_is, rollout_is_threshold)
    w = w.clamp(max=rollout_is_threshold).detach()
    if rollout_is_batch_normalize:
        dist_on = torch.distributed.is_available() and torch.distributed.is_initialized()
        if rollout_is == "token":
            mf = response_mask.to(w.dtype)
            mean = F_.distributed_masked_mean(w, mf) if dist_on else F_.masked_mean(w, response_mask)
        else:
            sw = F_.masked_mean(w, response_mask, axis=-1)
            sm = (response_mask.sum(dim=-1) > 0).to(w.dtype)
            mean = F_.distributed_masked_mean(sw, sm) if dist_on else (sw * sm).sum() / sm.sum().clamp_min(1e-8)
        if mean > 1e-8:
            w = w / mean
            metrics["rollout_is_batch_norm_factor"] = mean.item()
        else:
            metrics["rollout_is_batch_norm_factor"] = 1.0
    return w, metrics


def compute_offpolicy_metrics(old_log_prob: torch.Tensor, rollout_log_prob: Optional[torch.Tensor],
                              response_mask: torch.Tensor) -> dict[str, Any]:
    """KL / k3-KL / perplexities / log-PPL differences / chi-square between training and rollout policies."""
    assert response_mask.any(), "Expected at least one valid token in response_mask"
    m = {}
    lp_train = F_.masked_mean(old_log_prob, response_mask, axis=-1)
    m["training_ppl"] = torch.exp(-lp_train).mean().item()
    m["training_log_ppl"] = (-lp_train).mean().item()
    if rollout_log_prob is None:
        return m
    lr = old_log_prob - rollout_log_prob
    m["kl"] = F_.masked_mean(-lr, response_mask).item()
    m["k3_kl"] = F_.masked_mean(torch.exp(lr) - lr - 1, response_mask).item()
    lp_roll = F_.masked_mean(rollout_log_prob, response_mask, axis=-1)
    m["rollout_ppl"] = torch.exp(-lp_roll).mean().item()
    m["rollout_log_ppl"] = (-lp_roll).mean().item()
    d = lp_roll - lp_train
    m["log_ppl_diff"], m["log_ppl_abs_diff"] = d.mean().item(), d.abs().mean().item()
    m["log_ppl_diff_max"], m["log_ppl_diff_min"] = d.max().item(), d.min().item()
    m["ppl_ratio"] = torch.exp(d).mean().item()
    rho = torch.exp(torch.clamp(lr, min=-SAFETY_BOUND, max=SAFETY_BOUND))
    m["chi2_token"] = (F_.masked_mean(rho.square(), response_mask) - 1.0).item()
    lrs = torch.clamp(F_.masked_sum(lr, response_mask, axis=-1), min=-SAFETY_BOUND, max=SAFETY_BOUND)
    m["chi2_seq"] = (torch.exp(2.0 * lrs).mean() - 1.0).item()
    return m


def compute_rollout_correction_and_rejection_mask(old_log_prob: torch.Tensor, rollout_log_prob: torch.Tensor,
                                                  response_mask: torch.Tensor, rollout_is: Optional[str] = None,
                                                  rollout_is_threshold: Optional[float] = 2.0,
                                                  rollout_is_batch_normalize: bool = False,
                                                  rollout_rs: Optional[str] = None, rollout_rs_threshold=None):
    """Returns (DataProto{rollout_is_weights} | None, modified response_mask, {"rollout_corr/...": float})."""
    if not response_mask.any():
        raise ValueError("response_mask must contain at least one valid token (1).")
    if old_log_prob.shape != rollout_log_prob.shape:
        raise ValueError(f"old_log_prob shape {old_log_prob.shape} does not match rollout_log_prob shape {rollout_log_prob.shape}.")
    if old_log_prob.shape != response_mask.shape:
        raise ValueError(f"log_prob shape {old_log_prob.shape} does not match response_mask shape {response_mask.shape}.")
    log_ratio = old_log_prob - rollout_log_prob
    metrics: dict[str, float] = {}
    weights = None
    if rollout_is is not None and rollout_is_threshold is not None:
        weights, mm = compute_rollout_correction_weights(log_ratio, response_mask, rollout_is, rollout_is_threshold,
                                                         rollout_is_batch_normalize)
        metrics.update(mm)
    new_mask = response_mask.clone()
    if rollout_rs is not None:
        if rollout_rs_threshold is None:
            raise ValueError("rollout_rs_threshold must be explicitly provided when rollout_rs is enabled. "
                             "Set rollout_rs_threshold to the desired threshold value.")
        new_mask, mm = compute_rollout_rejection_mask(log_ratio, response_mask, rollout_rs, rollout_rs_threshold)
        metrics.update(mm)
    metrics.update(compute_offpolicy_metrics(old_log_prob, rollout_log_prob, response_mask))
    scalars = {f"rollout_corr/{k}": (v.item() if isinstance(v, torch.Tensor) else v) for k, v in metrics.items()}
    proto = DataProto.from_dict(tensors={"rollout_is_weights": weights}) if weights is not None else None
    return proto, new_mask, scalars


def _cfg_get(cfg, key, default=None):
    if cfg is None:
        return default
    if isinstance(cfg, dict):
        return cfg.get(key, default)
    if hasattr(cfg, "get"):
        return cfg.get(key, default)
    return getattr(cfg, key, default)


def compute_rollout_correction_and_add_to_batch(batch: DataProto, rollout_corr_config) -> tuple[DataProto, dict]:
    """Trainer entry: adds ``rollout_is_weights`` and replaces ``response_mask`` in the batch."""
    proto, new_mask, metrics = compute_rollout_correction_and_rejection_mask(
        old_log_prob=batch.batch["old_log_probs"], rollout_log_prob=batch.batch["rollout_log_probs"],
        response_mask=batch.batch["response_mask"], rollout_is=_cfg_get(rollout_corr_config, "rollout_is"),
        rollout_is_threshold=_cfg_get(rollout_corr_config, "rollout_is_threshold", 2.0),
        rollout_is_batch_normalize=_cfg_get(rollout_corr_config, "rollout_is_batch_normalize", False),
        rollout_rs=_cfg_get(rollout_corr_config, "rollout_rs"),
        rollout_rs_threshold=_cfg_get(rollout_corr_config, "rollout_rs_threshold"))
    batch.batch["response_mask"] = new_mask
    if proto is not None:
        batch = batch.union(proto)
    return batch, metrics


def compute_rollout_corr_metrics_from_logprobs(log_prob, rollout_log_prob, response_mask) -> dict[str, float]:
    return {f"rollout_corr/{k}": v for k, v in compute_offpolicy_metrics(log_prob, rollout_log_prob, response_mask).items()}


def apply_bypass_mode(batch: DataProto, rollout_corr_config=None, policy_loss_config=None) -> None:
    """Use the rollout log-probs as pi_old and route the actor to the ``bypass_mode`` policy loss."""
    if "rollout_log_probs" not in batch.batch:
        raise ValueError("bypass_mode=True requires rollout_log_probs in batch. Ensure rollout worker is configured to "
                         "calculate_log_probs=true.")
    batch.batch["old_log_probs"] = batch.batch["rollout_log_probs"]
    if policy_loss_config is not None:
        if isinstance(policy_loss_config, dict):
            policy_loss_config["rollout_correction"] = rollout_corr_config
            policy_loss_config["loss_mode"] = "bypass_mode"
        else:
            object.__setattr__(policy_loss_config, "rollout_correction", rollout_corr_config)
            object.__setattr__(policy_loss_config, "loss_mode", "bypass_mode")
