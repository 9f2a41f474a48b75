"""Code scoring through a Sandbox-Fusion HTTP service (verl/utils/reward_score/sandbox_fusion/).

Each test case runs the generated program with its stdin and compares stdout; the score is the fraction of
passed cases (``continuous=True``) or all-or-nothing. Calls are bounded by a semaphore and retried on
gateway time-outs.
"""

from __future__ import annotations

import json
import re
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Optional


def _extract_code(text: str) -> str:
    blocks = re.findall(r"```(?:python|py)?\n(.*?)```", text, re.DOTALL)
    return blocks[-1] if blocks else text


def call_sandbox_api(url: str, code: str, stdin: Optional[str], timeout: int = 10, memory_limit_mb: int = 1024,
                     language: str = "python", max_retries: int = 3):
    import requests

    payload = {"compile_timeout": timeout, "run_timeout": timeout, "code": code, "stdin": stdin, "language": language,
               "memory_limit_MB": memory_limit_mb, "files": {}, "fetch_files": []}
    err = None
    for attempt in range(max_retries):
        try:
            r = requests.post(url, headers={"Content-Type": "application/json", "Accept": "application/json"},
                              data=json.dumps(payload), timeout=timeout * 2 + 5)
            if r.status_code == 504:
                err = "gateway timeout"
                time.sleep(1.0 * (attempt + 1))
                continue
            r.raise_for_status()
            return r.json(), None
        except Exception as e:  # network errors are reported, not raised
            err = f"{type(e).__name__}: {e}"
            time.sleep(0.5 * (attempt + 1))
    return None, err


def _run_case(url, semaphore, code, stdin, expected, timeout, memory_limit_mb):
    if semaphore is not None:
        semaphore.acquire()
    try:
        resp, err = call_sandbox_api(url, code, stdin, timeout, memory_limit_mb)
    finally:
        if semaphore is not None:
            semaphore.release()
    if err or resp is None:
        return False, {"error": err}
    run = (resp.get("run_result") or {})
    ok = resp.get("status") == "Success" and (run.get("stdout") or "").strip() == str(expected).strip()
    return ok, {"status": resp.get("status"), "stdout": run.get("stdout"), "stderr": run.get("stderr")}


def compute_score(sandbox_fusion_url, concurrent_semaphore, memory_limit_mb, completion, test_cases, continuous=False,
                  timeout=10):
    code = _extract_code(completion)
    if isinstance(test_cases, str):
        test_cases = json.loads(test_cases)
    inputs, outputs = test_cases.get("inputs", []), test_cases.get("outputs", [])
    if not inputs:
        return 0.0, []
    with ThreadPoolExecutor(max_workers=min(len(inputs), 16)) as ex:
        res = list(ex.map(lambda io: _run_case(sandbox_fusion_url, concurrent_semaphore, code, io[0], io[1], timeout,
                                               memory_limit_mb or 1024), zip(inputs, outputs)))
    passed = sum(1 for ok, _ in res if ok)
    score = passed / len(inputs) if continuous else float(passed == len(inputs))
    return score, [m for _, m in res]
