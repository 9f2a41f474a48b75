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


def test_update_policy_with_sp_matches_dp_under_spmd_launch():
    """SPMD launch, 2 gloo ranks: update_actor with ulysses_sequence_parallel_size=2 (the ranks pool their shares)
    equals the data-parallel update over the same samples: loss, gradient norm, optimizer steps, weights."""
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29700 + os.getpid() % 250), os.path.join(here, "_sp_spmd_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "SP_SPMD_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])
