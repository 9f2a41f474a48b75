"""The benchmark entry point's contract that can be checked without a GPU: the reference arm answers with one JSON line
and exit code 0 whatever the state of the reference install, the argument defaults follow the benchmark configs, and the
composed trainer configs are the ones the lines claim."""

import json
import os
import subprocess
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_and_exits_zero():
    r = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                        "--warmup", "3"], capture_output=True, text=True, timeout=300, cwd=REPO)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip().startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and ("unavailable" in d or "value" in d)


def test_config_defaults_and_composition():
    sys.path.insert(0, REPO)
    try:
        import bench
    finally:
        sys.path.pop(0)
    old = sys.argv
    try:
        sys.argv = ["bench.py"]
        a = bench.parse_args()
        assert (a.gpus, a.config, a.prompts_per_gpu, a.n, a.max_response) == (1, 1, 16, 8, 1024) and a.steps >= 1 and a.warmup >= 3
        a.rollout_tp = 1
        c = bench.build_config(a, 8)
        assert c.data.train_batch_size == 128 and c.actor_rollout_ref.rollout.n == 8 and c.algorithm.adv_estimator == "grpo"
        assert c.actor_rollout_ref.actor.use_kl_loss and c.data.max_prompt_length == 512 and c.data.max_response_length == 1024
        sys.argv = ["bench.py", "--config", "2"]
        a = bench.parse_args()
        assert (a.prompts_per_gpu, a.n) == (32, 1)
        a.rollout_tp = 2
        c = bench.build_config(a, 8)
        assert c.data.train_batch_size == 256 and c.algorithm.adv_estimator == "gae" and c.critic.cliprange_value == 0.5
        assert c.actor_rollout_ref.rollout.tensor_model_parallel_size == 2 and c.algorithm.use_kl_in_reward
    finally:
        sys.argv = old
