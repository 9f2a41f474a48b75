"""PRIME-style math grading (verl/utils/reward_score/prime_math/): extract the final (boxed or last-number) answer and
grade it with the MATH normaliser, returning ``(is_correct, format_ok, extracted)`` as the reference does."""

from __future__ import annotations

import re

from . import math_reward


def _extract(solution: str):
    boxed = math_reward.last_boxed_only_string(solution) if hasattr(math_reward, "last_boxed_only_string") else None
    if boxed:
        try:
            return math_reward.remove_boxed(boxed), True
        except Exception:
            pass
    nums = re.findall(r"-?\d+(?:\.\d+)?(?:/\d+)?", solution.replace(",", ""))
    return (nums[-1], False) if nums else (None, False)


def compute_score(solution_str: str, ground_truth: str):
    ans, boxed = _extract(solution_str)
    if ans is None:
        return False, False, None
    norm = getattr(math_reward, "strip_string", lambda s: s.strip())
    try:
        ok = norm(str(ans)) == norm(str(ground_truth))
    except Exception:
        ok = str(ans).strip() == str(ground_truth).strip()
    if not ok:
        try:
            ok = abs(float(eval(str(ans), {"__builtins__": {}})) - float(eval(str(ground_truth), {"__builtins__": {}}))) < 1e-6
        except Exception:
            ok = False
    return bool(ok), boxed, ans
