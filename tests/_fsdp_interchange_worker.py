"""Child of tests/test_checkpoint_interchange_on_cpu.py: 2 gloo ranks save an engine as torch-FSDP style DTensor shard
files, a fresh engine loads them back, and a state dict sharded by torch's own ``distribute_tensor`` (what the reference
writes) loads as well."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    out = sys.argv[1]
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import DTensor, Shard, distribute_tensor

    from verl_b200.models import preset
    from verl_b200.models.hf_io import native_to_hf_state_dict
    from verl_b200.workers.engine.native import NativeEngine

    class C(dict):
        __getattr__ = dict.get

    cfg = preset("tiny-qwen2")
    eng = NativeEngine(cfg, C(), C(lr=1e-3), device="cpu", group=dist.group.WORLD, seed=3).initialize()
    full = {k: v.clone() for k, v in eng.zero.named_full_tensors()}
    eng.save_checkpoint(os.path.join(out, "a"), save_contents=("fsdp_model", "extra"))
    st = torch.load(os.path.join(out, "a", f"model_world_size_{world}_rank_{rank}.pt"), weights_only=False)
    assert "model.layers.0.self_attn.q_proj.weight" in st and isinstance(st["model.embed_tokens.weight"], DTensor)
    assert st["model.embed_tokens.weight"].placements == (Shard(0),)
    eng2 = NativeEngine(cfg, C(), C(lr=1e-3), device="cpu", group=dist.group.WORLD, seed=99).initialize()
    eng2.load_checkpoint(os.path.join(out, "a"), load_contents=("model",))
    for k, v in eng2.zero.named_full_tensors():
        torch.testing.assert_close(v, full[k])
    # a directory as the reference's FSDP2 engine writes it: torch shards the HF state dict itself
    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("fsdp",))
    hf = native_to_hf_state_dict(cfg, full)
    sd = {k: distribute_tensor(v.float(), mesh, [Shard(0)]) for k, v in hf.items()}
    os.makedirs(os.path.join(out, "b"), exist_ok=True)
    torch.save(sd, os.path.join(out, "b", f"model_world_size_{world}_rank_{rank}.pt"))
    if rank == 0:
        import json

        json.dump({"FSDP_version": 2, "world_size": world}, open(os.path.join(out, "b", "fsdp_config.json"), "w"))
        cfg.save_pretrained(os.path.join(out, "b", "huggingface"))
    dist.barrier()
    eng3 = NativeEngine(cfg, C(), C(lr=1e-3), device="cpu", group=dist.group.WORLD, seed=5).initialize()
    eng3.load_checkpoint(os.path.join(out, "b"))
    for k, v in eng3.zero.named_full_tensors():
        torch.testing.assert_close(v, full[k])
    if rank == 0:
        print("FSDP_INTERCHANGE_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
