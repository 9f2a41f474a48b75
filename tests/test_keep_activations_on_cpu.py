"""Keeping layer activations instead of recomputing them gives the same step (2 gloo ranks, ZeRO-3)."""

import os
import subprocess
import sys


def test_kept_activations_match_recomputation():
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29950 + os.getpid() % 300), os.path.join(here, "_keep_act_worker.py")]
    env = {k: v for k, v in os.environ.items() if k != "VERL_B200_KEEP_ACTIVATION_LAYERS"}
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "KEEP_ACT_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])
