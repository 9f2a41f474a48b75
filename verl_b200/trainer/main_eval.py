"""Offline evaluation of generated responses with the rule-based reward functions.

    python -m verl_b200.trainer.main_eval data.path=generation.jsonl data.response_key=responses

Role of verl/trainer/main_eval.py:1-80: every row's responses are scored with ``default_compute_score`` (or a
custom reward function), the mean score per ``data_source`` is printed as ``test_score/<source>``.
"""

from __future__ import annotations

import json
import sys
from collections import defaultdict

import numpy as np

from ..utils.config import compose_from_dict

DEFAULTS = {
    "data": {"path": None, "prompt_key": "prompt", "response_key": "responses", "data_source_key": "data_source",
             "reward_model_key": "reward_model"},
    "custom_reward_function": {"path": None, "name": "compute_score"},
}


def run_eval(config) -> dict:
    from ..trainer.ppo.reward import get_custom_reward_fn
    from ..utils.dataset.rl_dataset import _read_rows
    from ..utils.reward_score import default_compute_score

    fn = get_custom_reward_fn(config) or default_compute_score
    rows = _read_rows(config.data.path)
    by_source = defaultdict(list)
    for r in rows:
        src = r.get(config.data.data_source_key, "unknown")
        gt = (r.get(config.data.reward_model_key) or {}).get("ground_truth")
        scores = []
        for resp in r[config.data.response_key]:
            s = fn(src, resp, gt, r.get("extra_info"))
            scores.append(float(s["score"] if isinstance(s, dict) else s))
        by_source[src].append(float(np.mean(scores)) if scores else 0.0)
    out = {f"test_score/{k}": float(np.mean(v)) for k, v in by_source.items()}
    print(json.dumps(out))
    return out


def main(argv=None):
    cfg = compose_from_dict(DEFAULTS, list(sys.argv[1:] if argv is None else argv))
    run_eval(cfg)


if __name__ == "__main__":
    main()
