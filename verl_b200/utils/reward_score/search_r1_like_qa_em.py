"""Search-R1 style QA: exact match of the last ``<answer>...</answer>`` against any golden answer."""

import re
import string


def normalize_answer(s: str) -> str:
    s = s.lower()
    s = "".join(ch for ch in s if ch not in set(string.punctuation))
    s = re.sub(r"\b(a|an|the)\b", " ", s)
    return " ".join(s.split())


def em_check(prediction: str, golden_answers) -> int:
    if isinstance(golden_answers, str):
        golden_answers = [golden_answers]
    p = normalize_answer(prediction)
    return int(any(normalize_answer(g) == p for g in golden_answers))


def extract_solution(solution_str: str):
    m = list(re.finditer(r"<answer>(.*?)</answer>", solution_str, re.DOTALL))
    if len(m) < 1:
        return None
    return m[-1].group(1).strip()


def compute_score(solution_str, ground_truth, method="strict", format_score=0.0, score=1.0):
    ans = extract_solution(solution_str)
    if ans is None:
        return 0
    target = ground_truth["target"] if isinstance(ground_truth, dict) else ground_truth
    return score if em_check(ans, target) else format_score
