"""Child of tests/test_tp_training_on_cpu.py: 4 gloo ranks. Training with tensor_model_parallel_size = 2 (x 2 data
parallel, ZeRO over the ranks that hold the same slice) gives the log-probs, entropy, gradient norm and updated weights
of plain data-parallel training on the same samples: dense model with a vocabulary-parallel lm_head, tied embeddings,
and an MoE model with the experts split over the group."""
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
    lens = [9, 14, 6]
    cu = torch.tensor([0, 9, 23, 29], dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens])

    def sample(r, vocab):
        ids = torch.randint(0, vocab, (sum(lens),), generator=torch.Generator().manual_seed(7 + r))
        return PackedBatch(ids, pos, cu, max(lens)), torch.roll(ids, -1)

    for name, cfg in (("untied", preset("tiny-qwen2", tie_word_embeddings=False)), ("tied", preset("tiny-qwen2")),
                      ("moe", preset("tiny-qwen3-moe"))):
        rows = torch.arange(sum(lens))
        res = {}
        for tp in (1, 2):
            eng = NativeEngine(cfg, C(tensor_model_parallel_size=tp), optim, device="cpu", group=dist.group.WORLD, seed=4).initialize()
            # tp = 2: ranks (0, 1) and (2, 3) share their samples: both data-parallel groups train on shares 0 and 1;
            # tp = 1: four data-parallel ranks; ranks 2, 3 repeat shares 0, 1 so that the global batch is the same twice
            share = (rank // 2) if tp == 2 else (rank % 2)
            batch, labels = sample(share, cfg.vocab_size)
            denom = 2.0 if tp == 2 else 4.0
            with eng.train_mode():
                eng.optimizer_zero_grad()
                lp, ent = eng.forward_logprob(batch, rows, labels, 1.0)
                ((-lp.mean() + 0.01 * ent.mean()) / denom).backward()
                gn = float(eng.optimizer_step())
            full = {k: v.float().clone() for k, v in eng._merged_named_tensors()}
            res[tp] = (share, lp.detach().clone(), ent.detach().clone(), gn, full)
            assert eng.get_data_parallel_size() == 4 // tp and eng.mp_size == tp
        # same share -> same log-probs; the global batch of the tp = 1 run holds every sample twice with weight 1/4 each,
        # the tp = 2 run once with weight 1/2: same gradient
        lp1 = res[1][1] if res[1][0] == res[2][0] else None
        if lp1 is not None:
            torch.testing.assert_close(res[2][1], lp1, atol=2e-5, rtol=1e-4)
            torch.testing.assert_close(res[2][2], res[1][2], atol=2e-5, rtol=1e-4)
        assert abs(res[1][3] - res[2][3]) < 2e-4 * max(1.0, res[1][3]), (name, res[1][3], res[2][3])
        for k, v in res[1][4].items():
            d = (v - res[2][4][k]).abs()
            # AdamW normalises the step: rounding moves single elements by up to 2 lr where a gradient is next to zero
            assert float(d.max()) <= 2.1e-3 and float(d.mean()) < 2e-5, (name, k, float(d.max()), float(d.mean()))
    dist.barrier()
    if rank == 0:
        print("TP_TRAIN_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
