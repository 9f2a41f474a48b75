"""Token-rule rewards for synthetic-prompt benchmarks (no tokenizer files needed): the response arrives either
as token ids (``extra_info["response_ids"]``) or as space-separated integers."""

from __future__ import annotations


def _ids(solution_str, extra_info):
    if isinstance(extra_info, dict) and extra_info.get("response_ids") is not None:
        return [int(t) for t in extra_info["response_ids"]]
    return [int(t) for t in str(solution_str).split() if t.lstrip("-").isdigit()]


def even_fraction(solution_str, ground_truth=None, extra_info=None, threshold=None) -> float:
    """Fraction of response tokens with an even id (optionally thresholded to 0 / 1)."""
    ids = _ids(solution_str, extra_info)
    if not ids:
        return 0.0
    frac = sum(1 for t in ids if t % 2 == 0) / len(ids)
    if threshold is not None:
        return float(frac > threshold)
    return frac


def contains_token(solution_str, ground_truth=4242, extra_info=None) -> float:
    """1 if the response contains the given token id, else 0."""
    target = 4242 if ground_truth is None else int(ground_truth)
    return float(target in _ids(solution_str, extra_info))
