"""``math_verify``-based grading (verl/utils/reward_score/math_verify.py); falls back to the MATH normaliser when the
``math_verify`` package is not installed."""

from __future__ import annotations

from . import math_reward


def compute_score(model_output: str, ground_truth: str, timeout_score: float = 0.0) -> float:
    try:
        from math_verify.metric import math_metric
        from math_verify.parser import ExprExtractionConfig, LatexExtractionConfig

        verify = math_metric(gold_extraction_target=(LatexExtractionConfig(),),
                             pred_extraction_target=(ExprExtractionConfig(), LatexExtractionConfig()))
        try:
            score, _ = verify(["\\boxed{" + ground_truth + "}"], [model_output])
            return float(score)
        except Exception:
            return timeout_score
    except ImportError:
        return float(math_reward.compute_score(model_output, ground_truth))
