"""Advantage estimators, policy / value losses, KL penalties and KL controllers.

Public names, registries and formulas follow verl/trainer/ppo/core_algos.py (estimators :214-1006,
``agg_loss`` :1025-1080, policy losses :1159-2200, value loss :1799-1838, KL :1841-1902). The
implementations here are vectorised: group statistics use segment reductions over the inverse
index of ``np.unique(uid)`` instead of Python dictionaries, and scans use ``cumsum``/``flip``
where the recurrence allows. GPU fast paths (``ops.gae``, ``ops.grpo_advantage``,
``ops.ppo_loss_fused``) implement the same math in single kernels.
"""

from __future__ import annotations

from enum import Enum
from typing import Any, Callable, Optional

import numpy as np
import torch

from ...utils import torch_functional as F_
from ...utils.groupwise import group_index, group_mean_std

__all__ = [
    "register_adv_est", "get_adv_estimator_fn", "register_policy_loss", "get_policy_loss_fn", "AdvantageEstimator",
    "AdaptiveKLController", "FixedKLController", "get_kl_controller", "agg_loss", "kl_penalty", "kl_penalty_forward",
    "compute_value_loss", "compute_entropy_loss", "compute_policy_loss", "compute_rewards",
    "compute_pf_ppo_reweight_data",
]

PolicyLossFn = Callable[..., tuple[torch.Tensor, dict[str, Any]]]
POLICY_LOSS_REGISTRY: dict[str, PolicyLossFn] = {}
ADV_ESTIMATOR_REGISTRY: dict[str, Any] = {}


def register_policy_loss(name: str) -> Callable[[PolicyLossFn], PolicyLossFn]:
    def deco(fn: PolicyLossFn) -> PolicyLossFn:
        POLICY_LOSS_REGISTRY[name] = fn
        return fn

    return deco


def get_policy_loss_fn(name: str) -> PolicyLossFn:
    if name not in POLICY_LOSS_REGISTRY:
        raise ValueError(f"Unsupported loss mode: {name}. Supported modes are: {list(POLICY_LOSS_REGISTRY.keys())}")
    return POLICY_LOSS_REGISTRY[name]


class AdvantageEstimator(str, Enum):
    GAE = "gae"
    GRPO = "grpo"
    REINFORCE_PLUS_PLUS = "reinforce_plus_plus"
    REINFORCE_PLUS_PLUS_BASELINE = "reinforce_plus_plus_baseline"
    REMAX = "remax"
    RLOO = "rloo"
    OPO = "opo"
    GRPO_PASSK = "grpo_passk"
    GPG = "gpg"
    RLOO_VECTORIZED = "rloo_vectorized"
    GRPO_VECTORIZED = "grpo_vectorized"
    OPTIMAL_TOKEN_BASELINE = "optimal_token_baseline"
    TIR_OPTIMAL_TOKEN_BASELINE = "tir_optimal_token_baseline"


def _name(x) -> str:
    return x.value if isinstance(x, Enum) else x


def register_adv_est(name_or_enum):
    def deco(fn):
        name = _name(name_or_enum)
        if name in ADV_ESTIMATOR_REGISTRY and ADV_ESTIMATOR_REGISTRY[name] != fn:
            raise ValueError(f"Adv estimator {name} has already been registered: {ADV_ESTIMATOR_REGISTRY[name]} vs {fn}")
        ADV_ESTIMATOR_REGISTRY[name] = fn
        return fn

    return deco


def get_adv_estimator_fn(name_or_enum):
    name = _name(name_or_enum)
    if name not in ADV_ESTIMATOR_REGISTRY:
        raise ValueError(f"Unknown advantage estimator simply: {name}")
    return ADV_ESTIMATOR_REGISTRY[name]


# ------------------------------------------------------------------ KL controllers
class AdaptiveKLController:
    """beta <- beta * (1 + clip(kl/target - 1, -0.2, 0.2) * n / horizon)  (arXiv:1909.08593)."""

    def __init__(self, init_kl_coef, target_kl, horizon):
        self.value = init_kl_coef
        self.target = target_kl
        self.horizon = horizon

    def update(self, current_kl, n_steps):
        err = float(np.clip(current_kl / self.target - 1, -0.2, 0.2))
        self.value *= 1 + err * n_steps / self.horizon


class FixedKLController:
    def __init__(self, kl_coef):
        self.value = kl_coef

    def update(self, current_kl, n_steps):
        pass


def _get(cfg, key, default=None):
    if cfg is None:
        return default
    if isinstance(cfg, dict):
        return cfg.get(key, default)
    if hasattr(cfg, "get") and not hasattr(cfg, key):
        return cfg.get(key, default)
    val = getattr(cfg, key, default)
    return default if val is None else val


def get_kl_controller(kl_ctrl):
    typ = _get(kl_ctrl, "type", "fixed")
    if typ == "fixed":
        return FixedKLController(kl_coef=_get(kl_ctrl, "kl_coef", 0.001))
    if typ == "adaptive":
        horizon = _get(kl_ctrl, "horizon", 10000)
        assert horizon > 0, f"horizon must be larger than 0. Got {horizon}"
        return AdaptiveKLController(_get(kl_ctrl, "kl_coef", 0.001), _get(kl_ctrl, "target_kl", 0.1), horizon)
    raise NotImplementedError(typ)


# -------------------------------------------------------------- advantage estimators
def _broadcast(seq_vals: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    return seq_vals.unsqueeze(-1) * mask


def _reverse_cumsum(x: torch.Tensor) -> torch.Tensor:
    return x.flip(-1).cumsum(-1).flip(-1)


@register_adv_est(AdvantageEstimator.GAE)
def compute_gae_advantage_return(token_level_rewards: torch.Tensor, values: torch.Tensor,
                                 response_mask: torch.Tensor, gamma, lam, whiten: bool = True):
    """delta_t = r_t + gamma V_{t+1} - V_t ; A_t = delta_t + gamma lam A_{t+1}. Masked (tool /
    observation) tokens pass the running next-value and advantage through unchanged."""
    with torch.no_grad():
        if token_level_rewards.is_cuda:
            from ... import ops

            adv, returns = ops.gae(token_level_rewards, values, response_mask, float(gamma), float(lam))
        else:
            B, T = token_level_rewards.shape
            nextv = torch.zeros(B, dtype=values.dtype)
            last = torch.zeros(B, dtype=values.dtype)
            adv = torch.zeros_like(values)
            mask = response_mask.to(values.dtype)
            for t in range(T - 1, -1, -1):
                m = mask[:, t]
                delta = token_level_rewards[:, t] + gamma * nextv - values[:, t]
                cand = delta + gamma * lam * last
                nextv = values[:, t] * m + (1 - m) * nextv
                last = cand * m + (1 - m) * last
                adv[:, t] = last
            returns = adv + values
        if whiten:
            adv = F_.masked_whiten(adv, response_mask)
    return adv, returns


@register_adv_est(AdvantageEstimator.GRPO)
def compute_grpo_outcome_advantage(token_level_rewards: torch.Tensor, response_mask: torch.Tensor, index: np.ndarray,
                                   epsilon: float = 1e-6, norm_adv_by_std_in_grpo: bool = True, config=None, **kwargs):
    """(score - group mean) / (group std + eps); singleton groups use mean 0 / std 1."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        inv, n_groups = group_index(index, scores.device)
        if scores.is_cuda:
            from ... import ops

            adv = ops.grpo_advantage(scores, inv, response_mask, n_groups, epsilon, norm_adv_by_std_in_grpo)
            adv = adv.to(token_level_rewards.dtype)
        else:
            mean, std, _ = group_mean_std(scores, inv, n_groups)
            a = scores - mean
            if norm_adv_by_std_in_grpo:
                a = a / (std + epsilon)
            adv = _broadcast(a, response_mask)
    return adv, adv


@register_adv_est(AdvantageEstimator.GRPO_VECTORIZED)
def compute_grpo_vectorized_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6,
                                              norm_adv_by_std_in_grpo: bool = True, config=None, **kwargs):
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        inv, n_groups = group_index(index, scores.device)
        mean, std, _ = group_mean_std(scores, inv, n_groups)
        a = scores - mean
        if norm_adv_by_std_in_grpo:
            a = a / (std + epsilon)
        adv = _broadcast(a, response_mask)
    return adv, adv


@register_adv_est(AdvantageEstimator.GRPO_PASSK)
def compute_grpo_passk_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6,
                                         norm_adv_by_std_in_grpo: bool = True, config=None, **kwargs):
    """Pass@k: only the best response of a group is credited, with r_max - r_second_max."""
    if config is not None:
        norm_adv_by_std_in_grpo = _get(config, "norm_adv_by_std_in_grpo", True)
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        inv, n_groups = group_index(index, scores.device)
        counts = torch.bincount(inv, minlength=n_groups)
        if int(counts.min()) < 2:
            bad = int(torch.nonzero(counts < 2)[0])
            raise ValueError(f"Pass@k requires at least 2 samples per group. Got {int(counts[bad])} for group {bad}.")
        adv_seq = torch.zeros_like(scores)
        order = torch.argsort(inv, stable=True)
        starts = torch.cumsum(counts, 0) - counts
        for g in range(n_groups):
            members = order[starts[g] : starts[g] + counts[g]]
            r = scores[members]
            top, top_i = torch.topk(r, 2)
            a = top[0] - top[1]
            if norm_adv_by_std_in_grpo:
                a = a / (torch.std(r) + epsilon)
            adv_seq[members[top_i[0]]] = a
        adv = _broadcast(adv_seq, response_mask)
    return adv, adv


@register_adv_est(AdvantageEstimator.REINFORCE_PLUS_PLUS_BASELINE)
def compute_reinforce_plus_plus_baseline_outcome_advantage(token_level_rewards, response_mask, index,
                                                           epsilon: float = 1e-6, config=None, **kwargs):
    """Group-mean baseline, then whitening over all valid tokens of the batch."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        inv, n_groups = group_index(index, scores.device)
        mean, _, _ = group_mean_std(scores, inv, n_groups)
        s = _broadcast(scores - mean, response_mask)
        s = F_.masked_whiten(s, response_mask) * response_mask
    return s, s


@register_adv_est(AdvantageEstimator.RLOO)
def compute_rloo_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6, config=None,
                                   **kwargs):
    """Leave-one-out baseline: s_i - mean_{j != i} s_j; singleton groups keep their score."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        inv, n_groups = group_index(index, scores.device)
        cnt = torch.bincount(inv, minlength=n_groups)[inv].to(scores.dtype)
        tot = torch.zeros(n_groups, dtype=scores.dtype, device=scores.device).index_add_(0, inv, scores)[inv]
        multi = cnt > 1
        loo = (tot - scores) / (cnt - 1).clamp(min=1)
        a = torch.where(multi, scores - loo, scores)
        adv = _broadcast(a, response_mask)
    return adv, adv


@register_adv_est(AdvantageEstimator.RLOO_VECTORIZED)
def compute_rloo_vectorized_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6,
                                              config=None, **kwargs):
    """Same estimator; singleton groups get zero advantage (as in the reference's vectorised form)."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        inv, n_groups = group_index(index, scores.device)
        cnt = torch.bincount(inv, minlength=n_groups)[inv].to(scores.dtype)
        tot = torch.zeros(n_groups, dtype=scores.dtype, device=scores.device).index_add_(0, inv, scores)[inv]
        a = ((cnt * scores - tot) / (cnt - 1).clamp(min=1)) * (cnt > 1)
        adv = _broadcast(a, response_mask)
    return adv, adv


@register_adv_est(AdvantageEstimator.OPO)
def compute_opo_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6, config=None,
                                  **kwargs):
    """Length-weighted group baseline (arXiv:2505.23585)."""
    with torch.no_grad():
        lengths = response_mask.sum(dim=-1).to(token_level_rewards.dtype)
        scores = token_level_rewards.sum(dim=-1)
        inv, n_groups = group_index(index, scores.device)
        z = torch.zeros(n_groups, dtype=scores.dtype, device=scores.device)
        num = z.clone().index_add_(0, inv, lengths * scores)
        den = z.clone().index_add_(0, inv, lengths)
        cnt = torch.bincount(inv, minlength=n_groups)
        base = torch.where(cnt > 1, num / den.clamp(min=1e-12), torch.zeros_like(num))
        adv = _broadcast(scores - base[inv], response_mask)
    return adv, adv


@register_adv_est(AdvantageEstimator.REINFORCE_PLUS_PLUS)
def compute_reinforce_plus_plus_outcome_advantage(token_level_rewards, response_mask, config=None, **kwargs):
    """Discounted return-to-go (reset after the last valid token), whitened over the batch."""
    assert config is not None
    gamma = _get(config, "gamma", 1.0)
    with torch.no_grad():
        T = token_level_rewards.shape[1]
        returns = torch.zeros_like(token_level_rewards)
        running = torch.zeros_like(token_level_rewards[:, 0])
        for t in range(T - 1, -1, -1):
            running = token_level_rewards[:, t] + gamma * running
            returns[:, t] = running
            running = running * response_mask[:, t]
        adv = F_.masked_whiten(returns, response_mask) * response_mask
    return adv, returns


@register_adv_est(AdvantageEstimator.REMAX)
def compute_remax_outcome_advantage(token_level_rewards, reward_baselines, response_mask, config=None, **kwargs):
    """Return-to-go minus the reward of a greedy rollout of the same prompt (arXiv:2310.10505)."""
    with torch.no_grad():
        returns = _reverse_cumsum(token_level_rewards * response_mask)
        adv = returns - reward_baselines.unsqueeze(-1) * response_mask
    return adv, returns


@register_adv_est(AdvantageEstimator.GPG)
def compute_gpg_outcome_advantage(token_level_rewards, response_mask, index, epsilon: float = 1e-6,
                                  f_norm: float = 1.0, alpha: float = 1.0, config=None, **kwargs):
    """alpha * (score - group mean) / f_norm with alpha = batch / #non-zero scores."""
    with torch.no_grad():
        scores = token_level_rewards.sum(dim=-1)
        alpha = scores.shape[0] / torch.count_nonzero(scores).clamp(min=1)
        inv, n_groups = group_index(index, scores.device)
        mean, _, _ = group_mean_std(scores, inv, n_groups)
        adv = _broadcast(alpha * (scores - mean) / f_norm, response_mask)
    return adv, adv


def _zero_tail(baselines, rows, lengths):
    """Zero the baseline of the single longest trajectory beyond the second-longest length."""
    srt, _ = torch.sort(lengths)
    mx, second = int(srt[-1]), int(srt[-2])
    longest = torch.nonzero(lengths == mx, as_tuple=True)[0]
    if longest.numel() == 1 and mx > second:
        baselines[rows[int(longest[0])], second:] = 0.0


@register_adv_est(AdvantageEstimator.OPTIMAL_TOKEN_BASELINE)
def compute_optimal_token_baseline_advantage(token_level_rewards, response_mask, index, old_log_probs,
                                             sum_pi_squared, rollout_is_weights=None, handle_zero_tail: bool = False,
                                             epsilon: float = 1e-8, **kwargs):
    """Per-timestep baseline B_t = sum_i G_t W_t / sum_i W_t over the prompt group, with
    W_t = cumsum(1 - 2 pi_t + sum pi^2) the cumulative path-variance proxy."""
    with torch.no_grad():
        returns = _reverse_cumsum(token_level_rewards * response_mask)
        w = 1 - 2 * torch.exp(old_log_probs) + sum_pi_squared
        if rollout_is_weights is not None:
            w = w * rollout_is_weights ** 2
        wc = (w * response_mask).cumsum(dim=-1)
        inv, n_groups = group_index(index, returns.device)
        T = returns.shape[1]
        z = torch.zeros(n_groups, T, dtype=returns.dtype, device=returns.device)
        num = z.clone().index_add_(0, inv, returns * wc * response_mask)
        den = z.clone().index_add_(0, inv, wc * response_mask) + epsilon
        cnt = torch.bincount(inv, minlength=n_groups)
        base = (num / den)[inv] * (cnt[inv] > 1).unsqueeze(-1)
        if handle_zero_tail:
            lengths = response_mask.sum(-1)
            for g in torch.nonzero(cnt > 1).flatten().tolist():
                rows = torch.nonzero(inv == g).flatten()
                _zero_tail(base, rows, lengths[rows])
        adv = (returns - base) * response_mask
    return adv, returns


@register_adv_est(AdvantageEstimator.TIR_OPTIMAL_TOKEN_BASELINE)
def compute_multi_turn_optimal_token_baseline_advantage(token_level_rewards, response_mask, index, old_log_probs,
                                                        sum_pi_squared, rollout_is_weights=None,
                                                        handle_zero_tail: bool = True, epsilon: float = 1e-8, **kwargs):
    """OTB for multi-turn data: model tokens are compacted to the left (tool tokens dropped) before
    the per-step group baseline, then scattered back."""
    with torch.no_grad():
        returns = _reverse_cumsum(token_level_rewards * response_mask)
        w = 1 - 2 * torch.exp(old_log_probs) + sum_pi_squared
        if rollout_is_weights is not None:
            w = w * rollout_is_weights ** 2
        wc = (w * response_mask).cumsum(dim=-1)
        mask_b = response_mask.bool()
        lengths = mask_b.sum(-1)
        B = returns.shape[0]
        L = int(lengths.max()) if B else 0
        rank = (mask_b.cumsum(-1) - 1).clamp(min=0)
        rows = torch.arange(B, device=returns.device).unsqueeze(-1).expand_as(rank)
        cw = torch.zeros(B, L, dtype=wc.dtype, device=wc.device)
        cr = torch.zeros(B, L, dtype=returns.dtype, device=returns.device)
        cw[rows[mask_b], rank[mask_b]] = wc[mask_b]
        cr[rows[mask_b], rank[mask_b]] = returns[mask_b]
        live = lengths > 0
        inv, n_groups = group_index(index, returns.device)
        z = torch.zeros(n_groups, L, dtype=returns.dtype, device=returns.device)
        num = z.clone().index_add_(0, inv[live], (cr * cw)[live])
        den = z.clone().index_add_(0, inv[live], cw[live]) + epsilon
        cnt = torch.zeros(n_groups, dtype=torch.long, device=returns.device).index_add_(0, inv[live],
                                                                                       torch.ones_like(inv[live]))
        base = (num / den)[inv] * (cnt[inv] > 1).unsqueeze(-1) * live.unsqueeze(-1)
        if handle_zero_tail:
            for g in torch.nonzero(cnt > 1).flatten().tolist():
                members = torch.nonzero((inv == g) & live).flatten()
                _zero_tail(base, members, lengths[members])
        cadv = cr - base
        adv = torch.zeros_like(returns)
        adv[mask_b] = cadv[rows[mask_b], rank[mask_b]]
        adv = adv * response_mask
    return adv, returns


def compute_rewards(token_level_scores, old_log_prob, ref_log_prob, kl_ratio):
    return token_level_scores - (old_log_prob - ref_log_prob) * kl_ratio


# ----------------------------------------------------------------------- aggregation
def agg_loss(loss_mat: torch.Tensor, loss_mask: torch.Tensor, loss_agg_mode: str, dp_size: int = 1,
             batch_num_tokens: Optional[int] = None, global_batch_size: Optional[int] = None,
             loss_scale_factor: Optional[int] = None, **_unused) -> torch.Tensor:
    """Reduce a [B,T] loss matrix to a scalar.

    token-mean: masked sum / batch_num_tokens * dp_size (defaults: local token count, dp_size 1)
    seq-mean-token-sum / seq-mean-token-mean: per-sequence token sum / mean over sequences that
      have at least one valid token, summed and divided by global_batch_size * dp_size
    seq-mean-token-sum-norm: sum of all token sums / loss_scale_factor (default: T)
    """
    if loss_agg_mode == "token-mean":
        if batch_num_tokens is None:
            batch_num_tokens = loss_mask.sum()
        return F_.masked_sum(loss_mat, loss_mask) / batch_num_tokens * dp_size
    if loss_agg_mode in ("seq-mean-token-sum", "seq-mean-token-mean"):
        seq = F_.masked_sum(loss_mat, loss_mask, axis=-1)
        if loss_agg_mode == "seq-mean-token-mean":
            seq = seq / (loss_mask.sum(-1) + 1e-8)
        seq_mask = (loss_mask.sum(-1) > 0).to(loss_mat.dtype)
        if global_batch_size is None:
            global_batch_size = seq_mask.sum()
        return F_.masked_sum(seq, seq_mask) / global_batch_size * dp_size
    if loss_agg_mode == "seq-mean-token-sum-norm":
        seq = F_.masked_sum(loss_mat, loss_mask, axis=-1)
        if loss_scale_factor is None:
            loss_scale_factor = loss_mask.shape[-1]
        return seq.sum() / loss_scale_factor
    raise ValueError(f"Invalid loss_agg_mode: {loss_agg_mode}")


def _batch_info(config) -> dict:
    info = _get(config, "global_batch_info", None)
    return dict(info) if info else {}


def _clip_params(config, clip_ratio_low=None, clip_ratio_high=None, clip_ratio_c=None):
    base = _get(config, "clip_ratio", 0.2)
    lo = clip_ratio_low if clip_ratio_low is not None else _get(config, "clip_ratio_low", base)
    hi = clip_ratio_high if clip_ratio_high is not None else _get(config, "clip_ratio_high", base)
    c = clip_ratio_c if clip_ratio_c is not None else _get(config, "clip_ratio_c", 3.0)
    return lo, hi, c


def _metrics(**kw) -> dict:
    return {f"actor/{k}": (v.detach().item() if isinstance(v, torch.Tensor) else float(v)) for k, v in kw.items()}


# --------------------------------------------------------------------- policy losses
def compute_policy_loss(old_log_prob, log_prob, advantages, response_mask, cliprange=None, cliprange_low=None,
                        cliprange_high=None, clip_ratio_c=3.0, loss_agg_mode: str = "token-mean"):
    """Legacy functional form returning (pg_loss, pg_clipfrac, ppo_kl, pg_clipfrac_lower)."""
    assert clip_ratio_c > 1.0, f"The lower bound of the clip_ratio_c for dual-clip PPO should be greater than 1.0, but get the value: {clip_ratio_c}."
    lo = cliprange if cliprange_low is None else cliprange_low
    hi = cliprange if cliprange_high is None else cliprange_high
    nkl = torch.clamp(log_prob - old_log_prob, min=-20.0, max=20.0)
    ratio = torch.exp(nkl)
    ppo_kl = F_.masked_mean(-nkl, response_mask)
    l1 = -advantages * ratio
    l2 = -advantages * torch.clamp(ratio, 1 - lo, 1 + hi)
    clip1 = torch.maximum(l1, l2)
    clipfrac = F_.masked_mean(torch.gt(l2, l1).float(), response_mask)
    l3 = -advantages * clip_ratio_c
    clip2 = torch.min(l3, clip1)
    clipfrac_lower = F_.masked_mean(torch.gt(clip1, l3) * (advantages < 0).float(), response_mask)
    pg_losses = torch.where(advantages < 0, clip2, clip1)
    return agg_loss(pg_losses, response_mask, loss_agg_mode), clipfrac, ppo_kl, clipfrac_lower


@register_policy_loss("vanilla")
def compute_policy_loss_vanilla(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode: str = "token-mean",
                                config=None, rollout_is_weights=None, clip_ratio_low=None, clip_ratio_high=None,
                                clip_ratio_c=None):
    """PPO clipped objective with dual-clip for negative advantages (arXiv:1707.06347, 1912.09729)."""
    lo, hi, c = _clip_params(config, clip_ratio_low, clip_ratio_high, clip_ratio_c)
    assert c > 1.0, f"The lower bound of the clip_ratio_c for dual-clip PPO should be greater than 1.0, but get the value: {c}."
    nkl = torch.clamp(log_prob - old_log_prob, min=-20.0, max=20.0)
    ratio = torch.exp(nkl)
    ppo_kl = F_.masked_mean(-nkl, response_mask)
    l1 = -advantages * ratio
    l2 = -advantages * torch.clamp(ratio, 1 - lo, 1 + hi)
    clip1 = torch.maximum(l1, l2)
    clipfrac = F_.masked_mean(torch.gt(l2, l1).float(), response_mask)
    l3 = -advantages * c
    clip2 = torch.min(l3, clip1)
    clipfrac_lower = F_.masked_mean(torch.gt(clip1, l3) * (advantages < 0).float(), response_mask)
    pg_losses = torch.where(advantages < 0, clip2, clip1)
    if rollout_is_weights is not None:
        pg_losses = pg_losses * rollout_is_weights
    pg_loss = agg_loss(pg_losses, response_mask, loss_agg_mode, **_batch_info(config))
    return pg_loss, _metrics(pg_clipfrac=clipfrac, ppo_kl=ppo_kl, pg_clipfrac_lower=clipfrac_lower)


@register_policy_loss("gspo")
def compute_policy_loss_gspo(old_log_prob, log_prob, advantages, response_mask,
                             loss_agg_mode: str = "seq-mean-token-mean", config=None, rollout_is_weights=None):
    """Sequence-level importance ratio (geometric mean over tokens), token-level gradient (arXiv:2507.18071)."""
    lo, hi, _ = _clip_params(config)
    nkl = log_prob - old_log_prob
    seq_len = response_mask.sum(-1).clamp(min=1)
    nkl_seq = (nkl * response_mask).sum(-1) / seq_len
    log_ratio = torch.clamp(log_prob - log_prob.detach() + nkl_seq.detach().unsqueeze(-1), max=10.0)
    ratio = torch.exp(log_ratio)
    l1 = -advantages * ratio
    l2 = -advantages * torch.clamp(ratio, 1 - lo, 1 + hi)
    pg_losses = torch.maximum(l1, l2)
    if rollout_is_weights is not None:
        pg_losses = pg_losses * rollout_is_weights
    pg_loss = agg_loss(pg_losses, response_mask, "seq-mean-token-mean", **_batch_info(config))
    clipfrac = F_.masked_mean(torch.gt(l2, l1).float(), response_mask)
    ppo_kl = F_.masked_mean(-nkl, response_mask)
    return pg_loss, _metrics(pg_clipfrac=clipfrac, ppo_kl=ppo_kl, pg_clipfrac_lower=0.0)


@register_policy_loss("sapo")
def compute_policy_loss_sapo(old_log_prob, log_prob, advantages, response_mask,
                             loss_agg_mode: str = "seq-mean-token-mean", config=None, rollout_is_weights=None):
    """Soft gate sigmoid(tau (r - 1)) * 4 / tau instead of hard clipping; tau depends on the advantage sign."""
    tau_pos = torch.as_tensor(_get(config, "tau_pos", 1.0), dtype=advantages.dtype, device=advantages.device)
    tau_neg = torch.as_tensor(_get(config, "tau_neg", 1.05), dtype=advantages.dtype, device=advantages.device)
    nkl = torch.clamp(log_prob - old_log_prob, min=-20.0, max=20.0)
    ratio = torch.exp(nkl)
    taus = torch.where(advantages > 0, tau_pos, tau_neg)
    gates = torch.sigmoid(taus * (ratio - 1.0)) * (4.0 / taus)
    pg_losses = -gates * advantages
    if rollout_is_weights is not None:
        pg_losses = pg_losses * rollout_is_weights
    pg_loss = agg_loss(pg_losses, response_mask, "seq-mean-token-mean", **_batch_info(config))
    ppo_kl = F_.masked_mean(-nkl, response_mask)
    return pg_loss, _metrics(pg_clipfrac=0.0, ppo_kl=ppo_kl, pg_clipfrac_lower=0.0)


@register_policy_loss("gpg")
def compute_policy_loss_gpg(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode: str = "token-mean",
                            config=None, rollout_is_weights=None):
    pg_losses = -log_prob * advantages
    if rollout_is_weights is not None:
        pg_losses = pg_losses * rollout_is_weights
    return agg_loss(pg_losses, response_mask, loss_agg_mode, **_batch_info(config)), {}


@register_policy_loss("clip_cov")
def compute_policy_loss_clip_cov(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode: str = "token-mean",
                                 config=None, rollout_is_weights=None):
    """Clip-Cov: detach a random subset of tokens whose (advantage, log-prob) covariance lies in [lb, ub]."""
    pl = _get(config, "policy_loss", None)
    ratio_sel = _get(pl, "clip_cov_ratio", 0.0002)
    ub, lb = _get(pl, "clip_cov_ub", 5.0), _get(pl, "clip_cov_lb", 1.0)
    lo, hi, _ = _clip_params(config)
    assert ratio_sel > 0, "clip_ratio should be larger than 0."
    nkl = log_prob - old_log_prob
    ratio = torch.exp(nkl)
    ppo_kl = F_.masked_mean(-nkl, response_mask)
    l1 = -advantages * ratio
    l2 = -advantages * torch.clamp(ratio, 1 - lo, 1 + hi)
    valid = response_mask > 0
    clipped = (l2 > l1) & valid
    cov = (advantages - F_.masked_mean(advantages, response_mask)) * (
        log_prob.detach() - F_.masked_mean(log_prob.detach(), response_mask))
    cov = cov.masked_fill(~valid | clipped, float("-inf"))
    n_clip = max(int(ratio_sel * response_mask.sum().item()), 1)
    cand = torch.nonzero((cov < ub) & (cov > lb) & valid)
    corr = torch.ones_like(advantages)
    if len(cand) > 0:
        pick = cand[torch.randperm(len(cand))[: min(n_clip, len(cand))]]
        corr[pick[:, 0], pick[:, 1]] = 0
    clipfrac = F_.masked_mean((corr == 0).float(), response_mask)
    pg_losses = torch.maximum(l1, l2) * corr
    if rollout_is_weights is not None:
        pg_losses = pg_losses * rollout_is_weights
    pg_loss = agg_loss(pg_losses, response_mask, loss_agg_mode, **_batch_info(config))
    return pg_loss, _metrics(pg_clipfrac=clipfrac, ppo_kl=ppo_kl)


@register_policy_loss("kl_cov")
def compute_policy_loss_kl_cov(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode: str = "token-mean",
                               config=None, rollout_is_weights=None):
    """KL-Cov: add an |log-ratio| penalty to the top-covariance fraction of tokens."""
    pl = _get(config, "policy_loss", None)
    sel = _get(pl, "kl_cov_ratio", 0.0002)
    coef = _get(pl, "ppo_kl_coef", 1.0)
    assert sel > 0, "kl_cov_ratio should be larger than 0."
    nkl = log_prob - old_log_prob
    ratio = torch.exp(nkl)
    ppo_kl_abs = F_.masked_mean(nkl.abs(), response_mask)
    base = -advantages * ratio
    with_kl = base + coef * nkl.abs()
    valid = response_mask > 0
    n_valid = int(valid.sum())
    pick = torch.zeros_like(valid)
    if n_valid > 0:
        a = advantages[valid].detach()
        lp = log_prob[valid].detach()
        cov = (a - a.mean()) * (lp - lp.mean())
        k = max(1, int(n_valid * sel))
        top = torch.topk(cov, k, largest=True).indices
        flat_idx = torch.nonzero(valid.reshape(-1), as_tuple=True)[0][top]
        pick.view(-1)[flat_idx] = True
    pg_losses = torch.where(pick, with_kl, base)
    if rollout_is_weights is not None:
        pg_losses = pg_losses * rollout_is_weights
    pg_loss = agg_loss(pg_losses, response_mask, loss_agg_mode, **_batch_info(config))
    return pg_loss, _metrics(ppo_kl=ppo_kl_abs)


@register_policy_loss("geo_mean")
def compute_policy_loss_geo_mean(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode: str = "token-mean",
                                 config=None, rollout_is_weights=None):
    """GMPO: clip token log-ratios, then use their geometric mean as a sequence ratio (arXiv:2507.20673)."""
    lo, hi, _ = _clip_params(config)
    nkl = log_prob - old_log_prob
    ppo_kl = F_.masked_mean(-nkl, response_mask)
    sgn = torch.sign(advantages)
    clamped = torch.clamp(nkl, -lo, hi)
    chosen = sgn * torch.min(sgn * nkl, sgn * clamped)
    n = response_mask.sum(-1)
    ratio = torch.exp((chosen * response_mask).sum(-1) / (n + 1e-8))
    adv_seq = (advantages * response_mask).sum(-1) / (n + 1e-8)
    pg_losses = -adv_seq * ratio
    if rollout_is_weights is not None:
        seq_w = torch.exp((torch.log(rollout_is_weights + 1e-10) * response_mask).sum(-1) / (n + 1e-8))
        pg_losses = pg_losses * seq_w
    pg_loss = pg_losses.mean()
    was_clipped = torch.ne(nkl, clamped)
    clipfrac = F_.masked_mean((was_clipped & (advantages > 0)).float(), response_mask)
    clipfrac_lower = F_.masked_mean((was_clipped & (advantages < 0)).float(), response_mask)
    return pg_loss, _metrics(pg_clipfrac=clipfrac, ppo_kl=ppo_kl, pg_clipfrac_lower=clipfrac_lower)


@register_policy_loss("cispo")
def compute_policy_loss_cispo(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode: str = "token-mean",
                              config=None, rollout_is_weights=None):
    """CISPO: stop-gradient clipped IS weight times A log pi (arXiv:2506.13585)."""
    lo, hi, _ = _clip_params(config)
    nkl = torch.clamp(log_prob - old_log_prob, min=-20.0, max=20.0)
    ratio = torch.exp(nkl)
    ppo_kl = F_.masked_mean(-nkl, response_mask)
    clipped = torch.clamp(ratio, 1 - lo, 1 + hi)
    pg_losses = -clipped.detach() * advantages * log_prob
    clipfrac = F_.masked_mean((ratio != clipped).float(), response_mask)
    if rollout_is_weights is not None:
        pg_losses = pg_losses * rollout_is_weights
    pg_loss = agg_loss(pg_losses, response_mask, loss_agg_mode, **_batch_info(config))
    return pg_loss, _metrics(pg_clipfrac=clipfrac, ppo_kl=ppo_kl, pg_clipfrac_lower=0.0)


def compute_policy_loss_reinforce(rollout_log_prob, log_prob, advantages, response_mask,
                                  loss_agg_mode: str = "seq-mean-token-sum", config=None, rollout_is_weights=None):
    """REINFORCE with optional importance weights: -w A log pi (no clipping)."""
    assert config is not None, "ActorConfig must be provided for REINFORCE loss"
    pg_losses = -advantages * log_prob
    if rollout_is_weights is not None:
        pg_losses = pg_losses * rollout_is_weights
    pg_loss = agg_loss(pg_losses, response_mask, loss_agg_mode, **_batch_info(config))
    kl = F_.masked_mean(-(log_prob - rollout_log_prob), response_mask)
    return pg_loss, _metrics(ppo_kl=kl)


@register_policy_loss("bypass_mode")
def compute_policy_loss_bypass_mode(old_log_prob, log_prob, advantages, response_mask,
                                    loss_agg_mode: str = "token-mean", config=None, rollout_is_weights=None):
    """Bypass mode: ``old_log_prob`` is the rollout policy's log-prob. IS weights / rejection masks are
    computed here from (current, rollout); ``ppo_clip`` relies on the clipped ratio alone, ``reinforce``
    applies the weights explicitly."""
    from .rollout_corr_helper import compute_rollout_correction_and_rejection_mask

    assert config is not None, "config is required for bypass_mode loss"
    pl = _get(config, "policy_loss", None)
    rc = _get(pl, "rollout_correction", None)
    if rc is None:
        raise ValueError("rollout_correction config not found in policy_loss. When using loss_mode='bypass_mode', "
                         "ensure rollout_correction config is passed.")
    loss_type = _get(rc, "loss_type", "ppo_clip")
    with torch.no_grad():
        weights_proto, new_mask, rc_metrics = compute_rollout_correction_and_rejection_mask(
            old_log_prob=log_prob, rollout_log_prob=old_log_prob, response_mask=response_mask,
            rollout_is=_get(rc, "rollout_is", None), rollout_is_threshold=_get(rc, "rollout_is_threshold", 2.0),
            rollout_is_batch_normalize=_get(rc, "rollout_is_batch_normalize", False),
            rollout_rs=_get(rc, "rollout_rs", None), rollout_rs_threshold=_get(rc, "rollout_rs_threshold", None))
    w = weights_proto.batch["rollout_is_weights"] if weights_proto else None
    if loss_type == "reinforce":
        loss, metrics = compute_policy_loss_reinforce(old_log_prob, log_prob, advantages, new_mask, loss_agg_mode,
                                                      config, w)
    elif loss_type == "ppo_clip":
        loss, metrics = compute_policy_loss_vanilla(old_log_prob, log_prob, advantages, new_mask, loss_agg_mode, config,
                                                    None)
    else:
        raise ValueError(f"Invalid loss_type: {loss_type}. Must be 'reinforce' or 'ppo_clip'.")
    metrics.update(rc_metrics)
    return loss, metrics


# ------------------------------------------------------------- entropy / value / KL
def compute_entropy_loss(logits, response_mask, loss_agg_mode: str = "token-mean"):
    return agg_loss(F_.entropy_from_logits(logits), response_mask, loss_agg_mode)


def compute_value_loss(vpreds: torch.Tensor, returns: torch.Tensor, values: torch.Tensor, response_mask: torch.Tensor,
                       cliprange_value: float, loss_agg_mode: str = "token-mean"):
    """0.5 * max((v - R)^2, (clip(v, V_old +- eps) - R)^2) and the fraction of clipped tokens."""
    vclip = F_.clip_by_value(vpreds, values - cliprange_value, values + cliprange_value)
    l1 = (vpreds - returns) ** 2
    l2 = (vclip - returns) ** 2
    vf_loss = 0.5 * agg_loss(torch.max(l1, l2), response_mask, loss_agg_mode)
    clipfrac = F_.masked_mean(torch.gt(l2, l1).float(), response_mask)
    return vf_loss, clipfrac


def kl_penalty_forward(logprob: torch.Tensor, ref_logprob: torch.Tensor, kl_penalty: str) -> torch.Tensor:
    """k1 ('kl'), 'abs', k2 ('mse'), k3 ('low_var_kl') estimators (http://joschu.net/blog/kl-approx.html)."""
    if kl_penalty in ("kl", "k1"):
        return logprob - ref_logprob
    if kl_penalty == "abs":
        return (logprob - ref_logprob).abs()
    if kl_penalty in ("mse", "k2"):
        return 0.5 * (logprob - ref_logprob).square()
    if kl_penalty in ("low_var_kl", "k3"):
        d = torch.clamp(ref_logprob - logprob, min=-20, max=20)
        return torch.clamp(torch.exp(d) - d - 1, min=-10, max=10)
    if kl_penalty == "full":
        raise NotImplementedError
    raise NotImplementedError(kl_penalty)


def kl_penalty(logprob: torch.Tensor, ref_logprob: torch.Tensor, kl_penalty: str) -> torch.Tensor:
    """Estimators whose name ends in '+' return the value of the chosen estimator with the gradient of k2."""
    fwd = kl_penalty_forward(logprob, ref_logprob, kl_penalty.rstrip("+"))
    if not kl_penalty.endswith("+") or kl_penalty in ("mse", "k2"):
        return fwd
    k2 = kl_penalty_forward(logprob, ref_logprob, "k2")
    return k2 - k2.detach() + fwd.detach()


def compute_pf_ppo_reweight_data(data, reweight_method: str = "pow", weight_pow: float = 2.0):
    """PF-PPO: resample the batch (with replacement) with weights derived from the sequence scores."""
    with torch.no_grad():
        scores = data.batch["token_level_scores"].sum(dim=-1)
        if reweight_method == "pow":
            w = scores.abs().pow(weight_pow)
        elif reweight_method == "max_min":
            w = ((scores == scores.max()) | (scores == scores.min())).to(scores.dtype)
        elif reweight_method == "max_random":
            w = torch.where(scores == scores.max(), 0.4, 0.1).to(scores.dtype)
        else:
            raise ValueError(f"Unsupported reweight_method: {reweight_method}")
        w = torch.clamp(w + 1e-8, min=1e-8)
        idx = torch.multinomial(w, scores.shape[0], replacement=True)
    out = data.select_idxs(idx)
    n = scores.shape[0]
    idx_list = idx.tolist()
    out.meta_info = {k: ([v[i] for i in idx_list] if isinstance(v, list) and len(v) == n else v)
                     for k, v in data.meta_info.items()}
    return out
