"""Child of tests/test_context_parallel.py: 2 gloo ranks. Training with context_parallel_size = 2 (both ranks work on
the same samples, each on two zig-zag chunks of every sequence) gives the log-probs, entropy, gradient norm and updated
weights of plain data-parallel training on those samples, for a dense and an MoE model, with sequence lengths that
need padding to a multiple of 2 * cp."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    from verl_b200.models import preset
    from verl_b200.models.transformer import PackedBatch
    from verl_b200.workers.engine.native import NativeEngine

    class C(dict):
        __getattr__ = dict.get

    optim = C(lr=1e-3, weight_decay=0.01, clip_grad=1.0)
    lens = [9, 14, 6, 1]
    cu = torch.tensor([0, 9, 23, 29, 30], dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens])

    for name, cfg in (("dense", preset("tiny-qwen2")), ("moe", preset("tiny-qwen3-moe"))):
        ids = torch.randint(0, cfg.vocab_size, (sum(lens),), generator=torch.Generator().manual_seed(11))
        batch, labels = PackedBatch(ids, pos, cu, max(lens)), torch.roll(ids, -1)
        rows = torch.arange(sum(lens))[::2]  # a subset of the positions, as the response rows of an RL batch are
        res = {}
        for cp in (1, 2):
            eng = NativeEngine(cfg, C(context_parallel_size=cp), optim, device="cpu", group=dist.group.WORLD, seed=4).initialize()
            assert eng.mp_size == cp and eng.get_data_parallel_size() == 2 // cp
            # cp = 1: both data-parallel ranks hold the same sample with weight 1/2; cp = 2: one copy with weight 1
            denom = 2.0 if cp == 1 else 1.0
            with eng.train_mode():
                eng.optimizer_zero_grad()
                lp, ent = eng.forward_logprob(batch, rows, labels[rows], 1.0)
                ((-lp.mean() + 0.01 * ent.mean()) / denom).backward()
                gn = float(eng.optimizer_step())
            full = {k: v.float().clone() for k, v in eng._merged_named_tensors()}
            res[cp] = (lp.detach().clone(), ent.detach().clone(), gn, full)
        torch.testing.assert_close(res[2][0], res[1][0], atol=2e-5, rtol=1e-4)
        torch.testing.assert_close(res[2][1], res[1][1], atol=2e-5, rtol=1e-4)
        assert abs(res[1][2] - res[2][2]) < 2e-4 * max(1.0, res[1][2]), (name, res[1][2], res[2][2])
        for k, v in res[1][3].items():
            d = (v - res[2][3][k]).abs()
            assert float(d.max()) <= 2.1e-3 and float(d.mean()) < 2e-5, (name, k, float(d.max()), float(d.mean()))
    dist.barrier()
    if rank == 0:
        print("CP_TRAIN_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
