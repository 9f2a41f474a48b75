"""Expert-parallel MoE training (experts owned by ranks, token all-to-all, no gather of expert matrices), 2 gloo ranks."""

import os
import subprocess
import sys


def test_expert_parallel_training_matches_zero3(tmp_path):
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29850 + os.getpid() % 140), os.path.join(here, "_ep_train_worker.py"), str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "EP_TRAIN_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-5000:])
