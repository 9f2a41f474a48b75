"""PRIME-style code grading (verl/utils/reward_score/prime_code/): run the model's program on the test cases
(stdin/stdout pairs or assert-style functional tests) in a subprocess with a time limit; the score is the fraction
of passed tests (``continuous``) or all-or-nothing."""

from __future__ import annotations

import json
import os
import re
import subprocess
import sys
import tempfile


def _extract_code(text: str) -> str:
    blocks = re.findall(r"```(?:python)?\n(.*?)```", text, flags=re.S)
    return blocks[-1] if blocks else text


def _run(code: str, stdin: str, timeout: float):
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "prog.py")
        with open(path, "w") as f:
            f.write(code)
        try:
            r = subprocess.run([sys.executable, "-I", path], input=stdin, capture_output=True, text=True, timeout=timeout, cwd=d,
                               env={"PATH": os.environ.get("PATH", "")})
            return r.returncode, r.stdout
        except subprocess.TimeoutExpired:
            return -9, ""


def compute_score(solution_str: str, ground_truth, continuous: bool = False, timeout: float = 5.0):
    tests = json.loads(ground_truth) if isinstance(ground_truth, str) else ground_truth
    code = _extract_code(solution_str)
    results = []
    if "inputs" in tests and "outputs" in tests:
        for inp, out in zip(tests["inputs"], tests["outputs"]):
            rc, got = _run(code, inp if isinstance(inp, str) else "\n".join(map(str, inp)), timeout)
            want = out if isinstance(out, str) else "\n".join(map(str, out))
            results.append(rc == 0 and got.split() == want.split())
    elif "functional" in tests:
        rc, _ = _run(code + "\n\n" + tests["functional"], "", timeout)
        results.append(rc == 0)
    else:
        return 0.0, {"error": "no tests"}
    if not results:
        return 0.0, {"passed": 0, "total": 0}
    frac = sum(results) / len(results)
    score = frac if continuous else float(all(results))
    return score, {"passed": int(sum(results)), "total": len(results)}
