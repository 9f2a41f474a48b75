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
    if rank == 0:
        print("CKPT_ENGINE_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
