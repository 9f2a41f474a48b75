"""Batched MATH scoring (verl/utils/reward_score/math_batch.py) for the batch reward manager."""

from __future__ import annotations

from . import math_reward


def compute_score_batched(data_sources, solution_strs, ground_truths, extra_infos=None):
    return [float(math_reward.compute_score(s, g)) for s, g in zip(solution_strs, ground_truths)]
