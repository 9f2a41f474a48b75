"""Debug metrics: how far the rollout engine's token probabilities are from the trainer's
(verl/utils/debug/metrics.py ``calculate_debug_metrics``)."""

from __future__ import annotations

import torch


def calculate_token_list_diff(student: torch.Tensor, teacher: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    diff = ((student != teacher) & mask.bool()).sum(-1)
    return diff.float() / mask.sum(-1).clamp(min=1)


def calculate_debug_metrics(data) -> dict:
    """rollout-vs-actor probability differences over valid response tokens and their Pearson correlation."""
    rollout = torch.exp(data.batch["rollout_log_probs"].float())
    actor = torch.exp(data.batch["old_log_probs"].float())
    mask = (data.batch["response_mask"] if "response_mask" in data.batch.keys() else
            data.batch["attention_mask"][:, -data.batch["responses"].size(1):]).bool()
    r, a = rollout[mask], actor[mask]
    if r.numel() == 0:
        return {}
    d = (r - a).abs()
    out = {"training/rollout_probs_diff_valid": 1, "training/rollout_probs_diff_max": d.max().item(),
           "training/rollout_probs_diff_mean": d.mean().item(), "training/rollout_probs_diff_std": d.std().item() if d.numel() > 1 else 0.0}
    if r.numel() > 1:
        rc, ac = r - r.mean(), a - a.mean()
        denom = (rc.norm() * ac.norm()).clamp(min=1e-12)
        out["training/rollout_actor_probs_pearson_corr"] = (rc @ ac / denom).item()
    return out
