"""Step metrics: data statistics, timing, throughput, variance proxies, bootstrap validation metrics.

Metric names follow verl/trainer/ppo/metric_utils.py (``critic/score|rewards|advantages|returns/*``,
``response_length/*``, ``prompt_length/*``, ``timing_s/*``, ``timing_per_token_ms/*``,
``perf/throughput``, ``perf/total_num_tokens``, ``perf/time_per_step``).
"""

from __future__ import annotations

from collections import defaultdict
from functools import partial
from typing import Any, Callable

import numpy as np
import torch

from ...protocol import DataProto
from ...utils import torch_functional as F_


def reduce_metrics(metrics: dict[str, list[Any]]) -> dict[str, Any]:
    """Mean of each list; keys containing "max" / "min" reduce with max / min (verl/utils/metric/utils.py:25)."""
    from ...utils.metric import reduce_metrics as _rm

    return _rm(metrics)


def _compute_response_info(batch: DataProto) -> dict[str, Any]:
    R = batch.batch["responses"].shape[-1]
    pm = batch.batch["attention_mask"][:, :-R]
    rm = batch.batch["attention_mask"][:, -R:]
    return dict(response_mask=rm, prompt_length=pm.sum(-1).float(), response_length=rm.sum(-1).float())


def _stats(prefix: str, x: torch.Tensor) -> dict:
    return {f"{prefix}/mean": x.mean().item(), f"{prefix}/max": x.max().item(), f"{prefix}/min": x.min().item()}


def compute_data_metrics(batch: DataProto, use_critic: bool = True) -> dict[str, Any]:
    seq_score = batch.batch["token_level_scores"].sum(-1)
    seq_reward = batch.batch["token_level_rewards"].sum(-1)
    adv, ret = batch.batch["advantages"], batch.batch["returns"]
    R = batch.batch["responses"].shape[-1]
    max_prompt = batch.batch["attention_mask"].shape[-1] - R
    info = _compute_response_info(batch)
    pl, rl = info["prompt_length"], info["response_length"]
    mask = batch.batch["response_mask"].bool() if "response_mask" in batch.batch.keys() else info["response_mask"].bool()
    valid_adv, valid_ret = torch.masked_select(adv, mask), torch.masked_select(ret, mask)
    aborted = rl == 0
    non_ab = ~aborted
    m = {}
    m.update(_stats("critic/score", seq_score[non_ab] if non_ab.any() else seq_score))
    m.update(_stats("critic/rewards", seq_reward[non_ab] if non_ab.any() else seq_reward))
    m.update(_stats("critic/advantages", valid_adv))
    m.update(_stats("critic/returns", valid_ret))
    if use_critic:
        values = batch.batch["values"]
        valid_v = torch.masked_select(values, mask)
        var_ret = torch.var(valid_ret)
        m.update(_stats("critic/values", valid_v))
        m["critic/vf_explained_var"] = (1.0 - torch.var(valid_ret - valid_v) / (var_ret + 1e-5)).item()
    m.update(_stats("response_length", rl))
    m["response_length/clip_ratio"] = torch.eq(rl, R).float().mean().item()
    rl_ok = rl[non_ab]
    if rl_ok.numel():
        m.update(_stats("response_length_non_aborted", rl_ok))
        m["response_length_non_aborted/clip_ratio"] = torch.eq(rl_ok, R).float().mean().item()
    m["response/aborted_ratio"] = aborted.float().mean().item()
    m.update(_stats("prompt_length", pl))
    m["prompt_length/clip_ratio"] = torch.eq(pl, max_prompt).float().mean().item()
    if "__num_turns__" in batch.non_tensor_batch:
        nt = batch.non_tensor_batch["__num_turns__"]
        m.update({"num_turns/min": float(nt.min()), "num_turns/max": float(nt.max()), "num_turns/mean": float(nt.mean())})
    if "tool_call_counts" in batch.non_tensor_batch:
        tc = batch.non_tensor_batch["tool_call_counts"]
        m.update({"tool_call_counts/min": float(tc.min()), "tool_call_counts/max": float(tc.max()),
                  "tool_call_counts/mean": float(tc.mean())})
    return m


def compute_timing_metrics(batch: DataProto, timing_raw: dict[str, float]) -> dict[str, Any]:
    info = _compute_response_info(batch)
    n_prompt = torch.sum(info["prompt_length"]).item()
    n_resp = torch.sum(info["response_length"]).item()
    n_all = n_prompt + n_resp
    per_section = {"gen": n_resp, **{k: n_all for k in ("ref", "values", "adv", "update_critic", "update_actor")}}
    out = {f"timing_s/{k}": v for k, v in timing_raw.items()}
    out.update({f"timing_per_token_ms/{k}": timing_raw[k] * 1000 / max(per_section[k], 1)
                for k in set(per_section) & set(timing_raw)})
    return out


def compute_throughout_metrics(batch: DataProto, timing_raw: dict[str, float], n_gpus: int) -> dict[str, Any]:
    total = sum(batch.meta_info["global_token_num"])
    t = timing_raw["step"]
    return {"perf/total_num_tokens": total, "perf/time_per_step": t, "perf/throughput": total / (t * n_gpus)}


def compute_variance_proxy_metrics(batch: DataProto, gradient_norm: float | None = None) -> dict[str, float]:
    """Signal / variance proxies of the policy-gradient estimate from sequence-level advantages and weights."""
    m = {}
    if gradient_norm is None or "advantages" not in batch.batch.keys():
        return m
    mask = batch.batch["response_mask"].float()
    adv = batch.batch["advantages"]
    seq_adv = (adv * mask).sum(-1) / mask.sum(-1).clamp(min=1)
    w = batch.batch["rollout_is_weights"] if "rollout_is_weights" in batch.batch.keys() else torch.ones_like(adv)
    seq_w = (w * mask).sum(-1) / mask.sum(-1).clamp(min=1)
    g2 = float(gradient_norm) ** 2
    m["variance_proxy/proxy1_signal_strength"] = g2
    var1 = (seq_w * seq_adv).pow(2).mean().item()
    m["variance_proxy/proxy2_total_power"] = var1
    m["variance_proxy/proxy3_pure_noise"] = max(var1 - g2, 0.0) / max(len(seq_adv) - 1, 1)
    m["variance_proxy/expected_a_squared"] = seq_adv.pow(2).mean().item()
    m["variance_proxy/expected_w"] = seq_w.mean().item()
    return m


def bootstrap_metric(data: list[Any], subset_size: int, reduce_fns: list[Callable], n_bootstrap: int = 1000,
                     seed: int = 42) -> list[tuple[float, float]]:
    rng = np.random.RandomState(seed)
    idx = rng.choice(len(data), size=(n_bootstrap, subset_size), replace=True)
    out = []
    for fn in reduce_fns:
        vals = [fn([data[i] for i in row]) for row in idx]
        out.append((float(np.mean(vals)), float(np.std(vals))))
    return out


def calc_maj_val(data: list[dict[str, Any]], vote_key: str, val_key: str) -> float:
    votes = defaultdict(list)
    for d in data:
        votes[d[vote_key]].append(d[val_key])
    best = max(votes.items(), key=lambda kv: len(kv[1]))
    return best[1][0]


def process_validation_metrics(data_sources: list[str], sample_uids: list[str], infos_dict: dict[str, list[Any]],
                               seed: int = 42) -> dict[str, dict[str, dict[str, float]]]:
    """Per data source / variable: mean@N, std@N, best@k / worst@k (bootstrap), maj@k when ``pred`` exists."""
    by = defaultdict(lambda: defaultdict(lambda: defaultdict(list)))
    for i, (ds, uid) in enumerate(zip(data_sources, sample_uids)):
        for var, vals in infos_dict.items():
            by[ds][uid][var].append(vals[i])
    per_uid = defaultdict(lambda: defaultdict(dict))
    for ds, uids in by.items():
        for uid, vars_ in uids.items():
            for var, vals in vars_.items():
                if not vals or isinstance(vals[0], str):
                    continue
                n = len(vals)
                met = {f"mean@{n}": float(np.mean(vals))}
                if n > 1:
                    met[f"std@{n}"] = float(np.std(vals))
                    ns, k = [], 2
                    while k < n:
                        ns.append(k)
                        k *= 2
                    ns.append(n)
                    for k in ns:
                        (bm, bs), (wm, ws) = bootstrap_metric(vals, k, [np.max, np.min], seed=seed)
                        met[f"best@{k}/mean"], met[f"best@{k}/std"] = bm, bs
                        met[f"worst@{k}/mean"], met[f"worst@{k}/std"] = wm, ws
                        if vars_.get("pred") is not None and var != "pred":
                            pairs = [{"val": v, "pred": p} for v, p in zip(vals, vars_["pred"])]
                            (mm, ms), = bootstrap_metric(pairs, k, [partial(calc_maj_val, vote_key="pred", val_key="val")], seed=seed)
                            met[f"maj@{k}/mean"], met[f"maj@{k}/std"] = mm, ms
                per_uid[ds][uid][var] = met
    agg = defaultdict(lambda: defaultdict(lambda: defaultdict(list)))
    for ds, uids in per_uid.items():
        for uid, vars_ in uids.items():
            for var, met in vars_.items():
                for name, v in met.items():
                    agg[ds][var][name].append(v)
    return {ds: {var: {name: float(np.mean(v)) for name, v in mets.items()} for var, mets in vars_.items()}
            for ds, vars_ in agg.items()}
