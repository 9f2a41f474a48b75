"""Child of tests/test_hsdp_on_cpu.py: 4 gloo ranks. Hybrid sharding (fsdp_size = 2: two replicas of two shard ranks)
gives the same step as sharding over all four ranks; a checkpoint written under HSDP loads into the fully sharded
engine."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    out_dir = sys.argv[1]
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    from verl_b200.models import preset
    from verl_b200.models.transformer import PackedBatch
    from verl_b200.workers.engine.native import NativeEngine

    class C(dict):
        __getattr__ = dict.get

    cfg = preset("tiny-qwen2")
    optim = C(lr=1e-3, weight_decay=0.01, clip_grad=1.0)
    lens = [9, 14, 6]
    ids = torch.randint(0, cfg.vocab_size, (sum(lens),), generator=torch.Generator().manual_seed(7 + rank))
    cu = torch.tensor([0, 9, 23, 29], dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens])
    batch = PackedBatch(ids, pos, cu, max(lens))
    rows, labels = torch.arange(ids.numel()), torch.roll(ids, -1)
    res = {}
    for fs in (-1, 2):
        eng = NativeEngine(cfg, C(fsdp_size=fs), optim, device="cpu", group=dist.group.WORLD, seed=4).initialize()
        assert eng.zero.world == (4 if fs < 0 else 2) and eng.world == 4 and eng.get_data_parallel_size() == 4
        with eng.train_mode():
            eng.optimizer_zero_grad()
            lp, _ = eng.forward_logprob(batch, rows, labels, 1.0)
            (-lp.mean() / 4).backward()
            gn = float(eng.optimizer_step())
        full = {k: v.clone() for k, v in eng.zero.named_full_tensors()}
        res[fs] = (gn, full, float(lp.mean()))
        if fs == 2:
            eng.save_checkpoint(os.path.join(out_dir, "hsdp"))
    (g0, w0, l0), (g1, w1, l1) = res[-1], res[2]
    assert abs(l0 - l1) < 1e-5 and abs(g0 - g1) < 1e-4 * max(1.0, g0), (l0, l1, g0, g1)
    for k in w0:
        d = (w0[k].float() - w1[k].float()).abs()
        assert float(d.max()) <= 2.1e-3 and float((d > 2e-6).float().mean()) < 2e-3, (k, float(d.max()))
    # the HSDP checkpoint (2 shard files) restores the fully sharded engine (4 ranks) through the merge path
    eng = NativeEngine(cfg, C(), optim, device="cpu", group=dist.group.WORLD, seed=99).initialize()
    eng.load_checkpoint(os.path.join(out_dir, "hsdp"), load_contents=("model",))
    for k, v in eng.zero.named_full_tensors():
        torch.testing.assert_close(v.float(), w1[k].float(), atol=1e-6, rtol=1e-5)
    files = sorted(f for f in os.listdir(os.path.join(out_dir, "hsdp")) if f.startswith("model_world_size"))
    assert files == ["model_world_size_2_rank_0.pt", "model_world_size_2_rank_1.pt"], files
    if rank == 0:
        print("HSDP_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
