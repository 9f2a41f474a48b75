"""Training-side tensor parallelism (column / row parallel blocks, expert slices, vocabulary-parallel fused lm_head)
on 4 gloo ranks, and the merged statistics of the vocabulary-parallel lm_head against the unsharded op."""

import os
import subprocess
import sys


def test_tp2_dp2_training_matches_data_parallel():
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1",
           "--master-port", str(29250 + os.getpid() % 300), os.path.join(here, "_tp_train_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "TP_TRAIN_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-5000:])
