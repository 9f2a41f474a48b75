"""Checkpoint interchange with torch-FSDP shard files (the reference's on-disk format), 2 gloo ranks."""

import os
import subprocess
import sys


def test_fsdp_dtensor_shards_round_trip_and_merge(tmp_path):
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29650 + os.getpid() % 300), os.path.join(here, "_fsdp_interchange_worker.py"), str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "FSDP_INTERCHANGE_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])
    # the merger reads the torch-FSDP directory without a process group (DTensor shards unpickle in a plain process)
    from verl_b200.utils.checkpoint.native_checkpoint import merge_sharded_checkpoint

    full = merge_sharded_checkpoint(tmp_path / "b")
    assert full["layers.0.self_attn.qkv_proj.weight"].shape[0] > 0
