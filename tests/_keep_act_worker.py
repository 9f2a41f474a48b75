"""Child of tests/test_keep_activations_on_cpu.py: 2 gloo ranks (ZeRO-3, dp = 2); a step with recomputed
activations and steps with 1 / all layers' activations kept must give the same gradients and weights."""
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

    cfg = preset("tiny-qwen2")
    optim = C(lr=1e-2, weight_decay=0.01, clip_grad=1.0)
    lens = [9, 14, 6]
    ids = torch.randint(0, cfg.vocab_size, (sum(lens),), generator=torch.Generator().manual_seed(7 + rank))
    cu = torch.tensor([0, 9, 23, 29], dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens])
    batch = PackedBatch(ids, pos, cu, max(lens))
    rows = torch.arange(ids.numel())
    labels = torch.roll(ids, -1)
    outs = []
    for keep in ("0", "1", str(cfg.num_hidden_layers)):
        eng = NativeEngine(cfg, C(keep_activation_layers=keep), optim, device="cpu", group=dist.group.WORLD, seed=4).initialize()
        with eng.train_mode():
            eng.optimizer_zero_grad()
            for _ in range(2):  # two micro-batches: gradients accumulate in the shard
                lp, _ = eng.forward_logprob(batch, rows, labels, 1.0)
                (-lp.mean() / 2).backward()
            grad = eng.zero.grad.clone()
            gn = float(eng.optimizer_step())
        outs.append((grad, gn, eng.zero.shard16.clone()))
    for g, gn, w in outs[1:]:
        torch.testing.assert_close(g, outs[0][0], atol=1e-6, rtol=1e-5)
        assert abs(gn - outs[0][1]) < 1e-5 * max(1.0, outs[0][1])
        torch.testing.assert_close(w, outs[0][2], atol=1e-6, rtol=1e-5)
    assert float(outs[0][0].abs().sum()) > 0
    if rank == 0:
        print("KEEP_ACT_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
