"""Hybrid sharding (fsdp_size < world): shard groups x replicas, 4 gloo ranks."""

import os
import subprocess
import sys


def test_hybrid_sharding_matches_full_sharding(tmp_path):
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1",
           "--master-port", str(29150 + os.getpid() % 300), os.path.join(here, "_hsdp_worker.py"), str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "HSDP_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-5000:])
