"""Multi-GPU tests: peer-memory collectives, the one-launch reshard and a ZeRO step on >= 2 GPUs."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(what: str, nproc: int = 2, timeout: int = 600, env: dict | None = None):
    port = 29000 + (os.getpid() % 500)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "_mg_worker.py"), what]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env={**os.environ, **(env or {})})
    assert r.returncode == 0 and f"MG_WORKER_OK {what}" in r.stdout, (r.stdout[-3000:], r.stderr[-6000:])


@pytest.mark.parametrize("what", ["comm", "reshard", "zero", "ag_gemm", "gemm_rs", "moe_ep", "ulysses_a2a", "tp_allreduce"])
def test_two_ranks(what):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run(what, 2)


@pytest.mark.parametrize("what", ["comm", "reshard", "zero", "ag_gemm", "gemm_rs", "moe_ep", "ulysses_a2a", "tp_allreduce"])
def test_all_ranks(what):
    n = torch.cuda.device_count()
    if n <= 2:
        pytest.skip("needs more than 2 GPUs")
    _run(what, min(n, 8))


@pytest.mark.parametrize("what", ["comm", "zero", "gemm_rs", "moe_ep", "ulysses_a2a", "tp_allreduce"])
def test_two_ranks_with_launch_jitter(what):
    """The same checks on the race-hunting build of the library (``python -m verl_b200._build --jitter``): every
    block of the communication kernels and of the GEMM starts after a pseudo-random sleep of up to ~16 us, so that
    blocks and ranks reach their flags and peer loads in orders a quiet machine never produces. Results must not
    change (the checks compare against references, bit-exactly where the op is deterministic)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from verl_b200 import _build

    if not _build.lib_path("jitter").exists():
        _build.build(flavour="jitter")
    _run(what, 2, env={"VERL_B200_JITTER": "1"})


def test_tensor_parallel_rollout_replica_two_ranks():
    """A rollout replica sliced over 2 GPUs (fused all-reduce + RMSNorm over peer memory, CUDA graphs) generates what
    the whole model generates on one GPU: dense, replicated KV heads, expert-parallel MoE."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    port = 29500 + (os.getpid() % 400)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "_tp_rollout_worker.py"), "cuda"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "TP_ROLLOUT_OK" in r.stdout, (r.stdout[-3000:], r.stderr[-6000:])
