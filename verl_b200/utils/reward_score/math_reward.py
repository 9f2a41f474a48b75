"""MATH: compare the last ``\\boxed{...}`` of the response with the reference after string normalisation."""

import re


def last_boxed_only_string(s: str):
    idx = s.rfind("\\boxed")
    if "\\boxed " in s:
        return "\\boxed " + s.split("\\boxed ")[-1].split("$")[0]
    if idx < 0:
        idx = s.rfind("\\fbox")
        if idx < 0:
            return None
    depth, end = 0, None
    for i in range(idx, len(s)):
        if s[i] == "{":
            depth += 1
        elif s[i] == "}":
            depth -= 1
            if depth == 0:
                end = i
                break
    return None if end is None else s[idx : end + 1]


def remove_boxed(s: str) -> str:
    if s.startswith("\\boxed "):
        return s[len("\\boxed "):]
    left = "\\boxed{"
    assert s.startswith(left) and s.endswith("}"), s
    return s[len(left):-1]


def _fix_fracs(s: str) -> str:
    parts = s.split("\\frac")
    out = parts[0]
    for sub in parts[1:]:
        out += "\\frac"
        if sub and sub[0] == "{":
            out += sub
            continue
        if len(sub) < 2:
            return s
        a, b = sub[0], sub[1]
        if b != "{":
            out += "{" + a + "}{" + b + "}" + sub[2:]
        else:
            out += "{" + a + "}" + b + sub[2:]
    return out


def _fix_a_slash_b(s: str) -> str:
    parts = s.split("/")
    if len(parts) != 2:
        return s
    try:
        a, b = int(parts[0]), int(parts[1])
        if s == f"{a}/{b}":
            return "\\frac{" + str(a) + "}{" + str(b) + "}"
    except ValueError:
        pass
    return s


def _fix_sqrt(s: str) -> str:
    return re.sub(r"\\sqrt(\w)", r"\\sqrt{\1}", s)


def strip_string(s: str) -> str:
    s = s.replace("\n", "").replace("\\!", "").replace("\\\\", "\\").replace("tfrac", "frac").replace("dfrac", "frac")
    s = s.replace("\\left", "").replace("\\right", "").replace("^{\\circ}", "").replace("^\\circ", "")
    s = s.replace("\\$", "")
    if "\\text{ " in s:
        s = s.split("\\text{ ")[0]
    s = s.replace("\\%", "").replace("%", "").replace(" .", " 0.").replace("{.", "{0.")
    if not s:
        return s
    if s[0] == ".":
        s = "0" + s
    if len(s.split("=")) == 2 and len(s.split("=")[0]) <= 2:
        s = s.split("=")[1]
    s = _fix_sqrt(s).replace(" ", "")
    s = _fix_fracs(s)
    if s == "0.5":
        s = "\\frac{1}{2}"
    return _fix_a_slash_b(s)


def is_equiv(a, b) -> bool:
    if a is None and b is None:
        return True
    if a is None or b is None:
        return False
    try:
        return strip_string(a) == strip_string(b)
    except Exception:
        return a == b


def compute_score(solution_str, ground_truth) -> float:
    try:
        boxed = last_boxed_only_string(solution_str)
        if boxed is not None and is_equiv(remove_boxed(boxed), ground_truth):
            return 1.0
    except Exception:
        pass
    return 0.0
