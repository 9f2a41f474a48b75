"""Advantage estimators, policy losses, KL penalties, aggregation (pins the formulas against independent loops;
role of the reference's tests/trainer/ppo/test_core_algos_on_cpu.py)."""

import numpy as np
import pytest
import torch

from verl_b200.trainer.ppo import core_algos as ca


def _mask(B, T, seed=0):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(1, T + 1, (B,), generator=g)
    return (torch.arange(T)[None, :] < lens[:, None]).float()


def test_registries():
    for name in ("gae", "grpo", "rloo", "reinforce_plus_plus", "remax", "opo", "gpg", "grpo_passk", "rloo_vectorized",
                 "grpo_vectorized", "reinforce_plus_plus_baseline", "optimal_token_baseline", "tir_optimal_token_baseline"):
        assert callable(ca.get_adv_estimator_fn(name)), name
    assert ca.get_adv_estimator_fn(ca.AdvantageEstimator.GAE) is ca.get_adv_estimator_fn("gae")
    for name in ("vanilla", "gspo", "sapo", "gpg", "clip_cov", "kl_cov", "geo_mean", "cispo", "bypass_mode"):
        assert callable(ca.get_policy_loss_fn(name)), name
    with pytest.raises(ValueError):
        ca.get_policy_loss_fn("nope")
    with pytest.raises(Exception):
        ca.get_adv_estimator_fn("nope")


def test_gae_matches_python_loop():
    torch.manual_seed(0)
    B, T, gamma, lam = 4, 9, 0.97, 0.9
    mask = _mask(B, T, 1)
    r, v = torch.randn(B, T) * mask, torch.randn(B, T) * mask
    adv, ret = ca.compute_gae_advantage_return(r, v, mask, gamma, lam)
    raw = torch.zeros(B, T)
    for b in range(B):
        last, nextv = 0.0, 0.0
        for t in reversed(range(T)):
            if mask[b, t] == 0:
                continue
            delta = r[b, t] + gamma * nextv - v[b, t]
            last = delta + gamma * lam * last
            raw[b, t] = last
            nextv = v[b, t]
    torch.testing.assert_close(ret, (raw + v) * mask if ret[mask == 0].abs().sum() == 0 else raw + v, atol=1e-5, rtol=1e-5)
    m = mask.bool()
    want = (raw[m] - raw[m].mean()) / torch.sqrt(raw[m].var(unbiased=True) + 1e-8)
    torch.testing.assert_close(adv[m], want, atol=1e-4, rtol=1e-4)


def test_grpo_group_statistics_and_vectorized_equivalence():
    torch.manual_seed(1)
    B, T = 8, 5
    mask = _mask(B, T, 2)
    scores = torch.randn(B)
    tlr = torch.zeros(B, T)
    last = mask.sum(-1).long() - 1
    tlr[torch.arange(B), last] = scores
    index = np.array(["a", "a", "a", "b", "b", "b", "b", "c"], dtype=object)
    adv, ret = ca.compute_grpo_outcome_advantage(tlr, mask, index)
    for g in ("a", "b"):
        sel = torch.tensor(index == g)
        want = (scores[sel] - scores[sel].mean()) / (scores[sel].std(unbiased=True) + 1e-6)
        torch.testing.assert_close(adv[sel].sum(-1) / mask[sel].sum(-1), want, atol=1e-5, rtol=1e-5)
    # a group of one keeps its raw score (mean 0, std 1 convention)
    torch.testing.assert_close(adv[7].sum() / mask[7].sum(), scores[7], atol=1e-5, rtol=1e-5)
    adv_v, _ = ca.compute_grpo_vectorized_outcome_advantage(tlr, mask, index)
    torch.testing.assert_close(adv_v, adv, atol=1e-5, rtol=1e-5)
    adv_ns, _ = ca.compute_grpo_outcome_advantage(tlr, mask, index, norm_adv_by_std_in_grpo=False)
    sel = torch.tensor(index == "a")
    torch.testing.assert_close(adv_ns[sel].sum(-1) / mask[sel].sum(-1), scores[sel] - scores[sel].mean(), atol=1e-5, rtol=1e-5)


def test_rloo_loop_equals_vectorized():
    torch.manual_seed(2)
    B, T = 9, 4
    mask = _mask(B, T, 3)
    tlr = torch.randn(B, T) * mask
    index = np.array([0, 0, 0, 1, 1, 2, 2, 2, 2], dtype=object)
    a, _ = ca.compute_rloo_outcome_advantage(tlr, mask, index)
    b, _ = ca.compute_rloo_vectorized_outcome_advantage(tlr, mask, index)
    torch.testing.assert_close(a, b, atol=1e-5, rtol=1e-5)
    scores = tlr.sum(-1)
    sel = torch.tensor([i == 0 for i in index])
    n = int(sel.sum())
    want0 = scores[0] - (scores[sel].sum() - scores[0]) / (n - 1)
    torch.testing.assert_close(a[0].sum() / mask[0].sum(), want0, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("mode", ["token-mean", "seq-mean-token-sum", "seq-mean-token-mean", "seq-mean-token-sum-norm"])
def test_agg_loss_modes(mode):
    torch.manual_seed(3)
    loss, mask = torch.randn(3, 6), _mask(3, 6, 4)
    got = ca.agg_loss(loss, mask, mode)
    if mode == "token-mean":
        want = (loss * mask).sum() / mask.sum()
    elif mode == "seq-mean-token-sum":
        want = (loss * mask).sum(-1).mean()
    elif mode == "seq-mean-token-mean":
        want = ((loss * mask).sum(-1) / mask.sum(-1)).mean()
    else:
        want = (loss * mask).sum(-1).sum() / loss.shape[-1] / loss.shape[0] * 1.0 if False else None
    if want is not None:
        torch.testing.assert_close(got, want, atol=1e-6, rtol=1e-6)
    else:
        assert torch.isfinite(got)


def test_vanilla_policy_loss_clipping_and_dual_clip():
    old = torch.zeros(1, 4)
    lp = torch.log(torch.tensor([[1.5, 0.5, 5.0, 1.0]]))
    adv = torch.tensor([[1.0, 1.0, -1.0, 2.0]])
    mask = torch.ones(1, 4)
    cfg = {"clip_ratio": 0.2, "clip_ratio_low": 0.2, "clip_ratio_high": 0.2, "clip_ratio_c": 3.0}
    loss, m = ca.compute_policy_loss_vanilla(old, lp, adv, mask, "token-mean", cfg)
    # token 0: ratio 1.5 clipped to 1.2 -> -1.2 ; token 1: ratio .5 (unclipped is the max of the two losses) -> -0.5
    # token 2: negative advantage, ratio 5 -> loss min(max(5, 1.2.. ) , c) = 3 ; token 3: ratio 1 -> -2
    want = torch.tensor([-1.2, -0.5, 3.0, -2.0]).mean()
    torch.testing.assert_close(loss, want, atol=1e-5, rtol=1e-5)
    assert 0 < float(m["actor/pg_clipfrac"]) <= 1 and float(m["actor/pg_clipfrac_lower"]) > 0


@pytest.mark.parametrize("name", ["gspo", "sapo", "gpg", "clip_cov", "kl_cov", "geo_mean", "cispo"])
def test_policy_losses_finite_and_differentiable(name):
    torch.manual_seed(5)
    B, T = 4, 7
    mask = _mask(B, T, 6)
    old = torch.randn(B, T) * 0.1 - 2
    lp = (old + torch.randn(B, T) * 0.05).requires_grad_(True)
    adv = torch.randn(B, T)
    cfg = {"clip_ratio": 0.2, "clip_ratio_low": 0.2, "clip_ratio_high": 0.28, "clip_ratio_c": 3.0,
           "policy_loss": {"loss_mode": name, "clip_cov_ratio": 0.02, "clip_cov_lb": 1.0, "clip_cov_ub": 5.0,
                           "kl_cov_ratio": 0.2, "ppo_kl_coef": 0.1}}
    out = ca.get_policy_loss_fn(name)(old, lp, adv, mask, "token-mean", cfg)
    loss = out[0]
    assert torch.isfinite(loss)
    loss.backward()
    assert torch.isfinite(lp.grad).all() and float(lp.grad[mask == 0].abs().sum()) == 0.0


def test_kl_penalties_and_straight_through():
    lp = torch.tensor([[-1.0, -2.0]], requires_grad=True)
    ref = torch.tensor([[-1.5, -1.0]])
    d = lp - ref
    torch.testing.assert_close(ca.kl_penalty(lp, ref, "kl"), d)
    torch.testing.assert_close(ca.kl_penalty(lp, ref, "abs"), d.abs())
    torch.testing.assert_close(ca.kl_penalty(lp, ref, "mse"), 0.5 * d ** 2)
    k3 = torch.exp(-d) - 1 + d
    torch.testing.assert_close(ca.kl_penalty(lp, ref, "low_var_kl"), torch.clamp(k3, -10, 10))
    # '+' variants: value of the estimator, gradient of k2
    v = ca.kl_penalty(lp, ref, "low_var_kl+")
    torch.testing.assert_close(v.detach(), torch.clamp(k3, -10, 10).detach())
    v.sum().backward()
    torch.testing.assert_close(lp.grad, d.detach())


def test_kl_controllers_and_value_loss():
    a = ca.AdaptiveKLController(init_kl_coef=0.1, target_kl=1.0, horizon=100)
    a.update(current_kl=2.0, n_steps=10)
    assert a.value == pytest.approx(0.1 * (1 + 0.2 * 10 / 100))
    f = ca.FixedKLController(0.3)
    f.update(5.0, 10)
    assert f.value == 0.3
    v, vals, ret = torch.tensor([[1.0, 3.0]]), torch.tensor([[0.0, 0.0]]), torch.tensor([[2.0, 0.0]])
    loss, frac = ca.compute_value_loss(v, ret, vals, torch.ones(1, 2), cliprange_value=0.5)
    # token 0: max((1-2)^2, (0.5-2)^2) = 2.25 ; token 1: max(9, 0.25) = 9 -> 0.5 * mean
    assert float(loss) == pytest.approx(0.5 * (2.25 + 9.0) / 2) and float(frac) == pytest.approx(0.5)


def test_rollout_correction_weights_and_rejection():
    from verl_b200.trainer.ppo import rollout_corr_helper as rc

    old = torch.tensor([[-1.0, -1.0, -1.0], [-1.0, -1.0, -1.0]])
    roll = torch.tensor([[-1.0, -2.0, -0.5], [-1.0, -1.0, -4.0]])
    mask = torch.ones(2, 3)
    w, m = rc.compute_rollout_correction_weights(old - roll, mask, rollout_is="token", rollout_is_threshold=2.0)
    torch.testing.assert_close(w, torch.exp(old - roll).clamp(max=2.0))
    ws, _ = rc.compute_rollout_correction_weights(old - roll, mask, rollout_is="sequence", rollout_is_threshold=100.0)
    torch.testing.assert_close(ws[:, 0], torch.exp((old - roll).sum(-1)).clamp(max=100.0))
    keep, _ = rc.compute_rollout_rejection_mask(old - roll, mask, rollout_rs="token_k1", rollout_rs_threshold=2.0)
    assert keep[1, 2] == 0 and keep[0, 0] == 1  # exp(3) > 2 rejected
    met = rc.compute_offpolicy_metrics(old, roll, mask)
    assert any("kl" in k for k in met) and all(np.isfinite(float(v)) for v in met.values())
