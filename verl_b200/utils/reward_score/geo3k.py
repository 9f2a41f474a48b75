"""geometry3k: accuracy of the boxed answer (0.9) plus a think/boxed format bonus (0.1)."""

import re

from .math_reward import is_equiv, last_boxed_only_string, remove_boxed

_FORMAT = re.compile(r"<think>.*</think>.*\\boxed\{.*\}.*", re.DOTALL)


def format_reward(predict_str: str) -> float:
    return 1.0 if _FORMAT.fullmatch(predict_str) else 0.0


def acc_reward(predict_str: str, ground_truth: str, use_boxed: bool = True) -> float:
    if not use_boxed:  # the tool hands over the bare answer
        try:
            return 1.0 if is_equiv(predict_str.strip(), ground_truth) else 0.0
        except Exception:
            return 0.0
    boxed = last_boxed_only_string(predict_str)
    if boxed is None:
        return 0.0
    try:
        return 1.0 if is_equiv(remove_boxed(boxed), ground_truth) else 0.0
    except Exception:
        return 0.0


def compute_score(predict_str: str, ground_truth: str, use_boxed: bool = True, format_score: float = 0.1) -> float:
    return (1.0 - format_score) * acc_reward(predict_str, ground_truth, use_boxed) + format_score * format_reward(predict_str)
