"""DAPO math rule: ``Answer: <x>`` on the last lines (or the last boxed expression), score +1 / -1."""

import re

from .math_reward import last_boxed_only_string, remove_boxed

_SUBS = [("an ", ""), ("a ", ""), (".$", "$"), ("\\$", ""), (r"\ ", ""), (" ", ""), ("mbox", "text"),
         (",\\text{and}", ","), ("\\text{and}", ","), ("\\text{m}", "\\text{}")]
_REMOVED = ["square", "ways", "integers", "dollars", "mph", "inches", "hours", "km", "units", "\\ldots", "sue", "points",
            "feet", "minutes", "digits", "cents", "degrees", "cm", "gm", "pounds", "meters", "meals", "edges", "students",
            "childrentickets", "multiples", "\\text{s}", "\\text{.}", "\\text{\ns}", "\\text{}^2", "\\text{}^3", "\\text{\n}",
            "\\text{}", r"\mathrm{th}", r"^\circ", r"^{\circ}", r"\;", r",\!", "{,}", '"', "\\dots"]


def normalize_final_answer(ans: str) -> str:
    ans = ans.split("=")[-1]
    for a, b in _SUBS:
        ans = ans.replace(a, b)
    for r in _REMOVED:
        ans = ans.replace(r, "")
    ans = re.sub(r"(.*?)(\$)(.*?)(\$)(.*)", "$\\3$", ans)
    for pat in (r"(\\text\{)(.*?)(\})", r"(\\textbf\{)(.*?)(\})", r"(\\overline\{)(.*?)(\})", r"(\\boxed\{)(.*)(\})"):
        ans = re.sub(pat, "\\2", ans)
    ans = re.sub(r"(frac)([^{])(.)", "frac{\\2}{\\3}", ans)
    ans = re.sub(r"(sqrt)([^{])", "sqrt{\\2}", ans)
    ans = ans.replace("$", "")
    if ans.replace(",", "").isdigit():
        ans = ans.replace(",", "")
    return ans.strip()


def is_correct_minerva(solution_str: str, gt: str, gt_need_extract: bool = False,
                       answer_pattern: str = r"(?i)Answer\s*:\s*([^\n]+)"):
    m = re.findall(answer_pattern, solution_str)
    pred = normalize_final_answer(m[-1]) if m else "[INVALID]"
    if gt_need_extract:
        gt = normalize_final_answer(remove_boxed(last_boxed_only_string(gt)))
    else:
        gt = normalize_final_answer(gt)
    return pred == gt, pred


def is_correct_strict_box(pred: str, gt: str, pause_tokens_index=None):
    pred = pred[-100:]
    boxed = last_boxed_only_string(pred)
    extracted = remove_boxed(boxed) if boxed is not None else None
    return (1 if extracted == gt else -1), extracted


def verify(solution_str: str, answer: str, strict_box_verify: bool = False, pause_tokens_index=None):
    if strict_box_verify:
        c, pred = is_correct_strict_box(solution_str, answer, pause_tokens_index)
        return c == 1, pred
    return is_correct_minerva(solution_str, answer)


def compute_score(solution_str: str, ground_truth: str, strict_box_verify: bool = False, pause_tokens_index=None):
    solution_str = solution_str[-300:]
    correct, pred = verify(solution_str, ground_truth, strict_box_verify, pause_tokens_index)
    return {"score": 1.0 if correct else -1.0, "acc": bool(correct), "pred": pred}
