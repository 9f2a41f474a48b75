"""Pipeline parallelism (stages exchange the residual stream with send / recv autograd functions), 4 gloo ranks."""

import os
import subprocess
import sys


def test_pipeline_parallel_training_matches_data_parallel():
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1",
           "--master-port", str(29050 + os.getpid() % 300), os.path.join(here, "_pp_train_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "PP_TRAIN_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-5000:])
