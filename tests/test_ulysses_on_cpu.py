"""Ulysses sequence parallelism on 2 gloo ranks: a decoder layer gives the same outputs and gradients with the
sequence sharded (role of the reference's tests/models/test_transformers_ulysses.py)."""

import os
import subprocess
import sys


def test_ulysses_layer_matches_unsharded():
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29600 + os.getpid() % 300), os.path.join(here, "_ulysses_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "ULYSSES_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])
