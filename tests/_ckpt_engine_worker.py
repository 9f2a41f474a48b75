"""Child of tests/test_checkpoint_engine_on_cpu.py: rank 0 = trainer, ranks 1.. = rollout replicas (gloo)."""
import asyncio
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from verl_b200.checkpoint_engine import CheckpointEngineRegistry
    from verl_b200.models import preset
    from verl_b200.models.transformer import CausalLM

    cfg = preset("tiny-qwen2")
    tr, ro = CheckpointEngineRegistry.get("nccl").build_topology(1, world - 1, [])
    assert tr["rank"] == [0] and ro["rank"] == list(range(1, world))
    eng = CheckpointEngineRegistry.new("nccl", bucket_size=3 << 20, group=dist.group.WORLD, is_master=rank == 0, src=0,
                                       device=torch.device("cpu"))
    eng.prepare()
    ref = CausalLM(cfg, dtype=torch.float32, device="cpu")
    ref.init_weights(11)  # the trainer's weights; replicas start from something else
    if rank == 0:
        asyncio.run(eng.send_weights((k, v) for k, v in ref.state_dict().items()))
    else:
        model = CausalLM(cfg, dtype=torch.float32, device="cpu")
        model.init_weights(99)

        async def recv():
            got = {}
            async for name, t in eng.receive_weights():
                got[name] = t.clone()  # the bucket is reused by the next broadcast
            return got

        got = asyncio.run(recv())
        model.load_state_dict(got, strict=True)
        for k, v in ref.state_dict().items():
            assert torch.equal(model.state_dict()[k], v), k
    eng.finalize()
    dist.barrier()

    # pinned-host bucket engine with its overlap thread: ranks 0 and 1 are trainer ranks that own alternate buckets,
    # every rank consumes every bucket; a second version overwrites the first
    pe = CheckpointEngineRegistry.new("pinned_async", bucket_size=1 << 20, rank=rank, trainer_ranks=[0, 1],
                                      group=dist.group.WORLD, device="cpu")
    info = [(k, tuple(v.shape), v.dtype) for k, v in ref.state_dict().items()]
    buckets = pe.register(info)
    assert len(buckets) >= 2 and {b.owner for b in buckets} == {0, 1}
    assert set(pe.host) == ({i for i, b in enumerate(buckets) if b.owner == rank} if rank < 2 else set())
    for version in (1, 2):
        src = {k: v + float(version) for k, v in ref.state_dict().items()}
        if rank < 2:
            pe.stage(src, version=version)
        got = {}
        order = []

        def consume(pairs):
            order.append(len(pairs))
            for n, t in pairs:
                got[n] = t.clone()

        nbytes = pe.publish(consume)
        assert nbytes == sum(b.nbytes for b in buckets) and len(order) == len(buckets)
        for k, v in src.items():
            assert torch.equal(got[k], v), (version, k)
    pe.finalize()
    dist.barrier()
    if rank == 0:
        print("CKPT_ENGINE_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
