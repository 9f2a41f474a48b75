"""GSM8K: the final answer follows ``####`` (strict) or is the last number in the text (flexible)."""

import re

_STRICT = re.compile(r"#### (\-?[0-9\.\,]+)")
_NUMBER = re.compile(r"(\-?[0-9\.\,]+)")
_CLIP = 300


def extract_solution(solution_str: str, method: str = "strict"):
    assert method in ("strict", "flexible")
    if len(solution_str) > _CLIP:
        solution_str = solution_str[-_CLIP:]
    if method == "strict":
        found = _STRICT.findall(solution_str)
        return found[-1].replace(",", "").replace("$", "") if found else None
    for cand in reversed(_NUMBER.findall(solution_str)):
        if cand not in ("", "."):
            return cand
    return None


def compute_score(solution_str, ground_truth, method="strict", format_score=0.0, score=1.0):
    ans = extract_solution(solution_str, method)
    if ans is None:
        return 0
    return score if ans == ground_truth else format_score
