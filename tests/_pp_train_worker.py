"""Child of tests/test_pp_training_on_cpu.py: 4 gloo ranks. Pipeline parallelism (2 stages x 2 data-parallel ranks,
and 2 stages x tensor-parallel 2) gives the log-probs, gradient norm and updated weights of plain data-parallel
training on the same samples, through the per-micro-batch interface and through the pipelined batch interface."""
import os
import sys
from functools import partial

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    from verl_b200.models import preset
    from verl_b200.models.transformer import PackedBatch
    from verl_b200.utils import tensordict_utils as tu
    from verl_b200.workers.engine.native import NativeEngine
    from verl_b200.workers.utils.losses import sft_loss_on_batch

    class C(dict):
        __getattr__ = dict.get

    optim = C(lr=1e-3, weight_decay=0.01, clip_grad=1.0)
    cfg = preset("tiny-qwen2", tie_word_embeddings=False, num_hidden_layers=3)
    lens = [9, 14, 6]
    cu = torch.tensor([0, 9, 23, 29], dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens])
    rows = torch.arange(sum(lens))

    def sample(r):
        ids = torch.randint(0, cfg.vocab_size, (sum(lens),), generator=torch.Generator().manual_seed(7 + r))
        return PackedBatch(ids, pos, cu, max(lens)), torch.roll(ids, -1), ids

    def step(ec, share, denom):
        eng = NativeEngine(cfg, ec, optim, device="cpu", group=dist.group.WORLD, seed=4).initialize()
        batch, labels, _ = sample(share)
        with eng.train_mode():
            eng.optimizer_zero_grad()
            lp, ent = eng.forward_logprob(batch, rows, labels, 1.0)
            ((-lp.mean() + 0.01 * ent.mean()) / denom).backward()
            gn = float(eng.optimizer_step())
        full = {k: v.float().clone() for k, v in eng._merged_named_tensors()}
        return eng, lp.detach().clone(), gn, full

    # reference: 4 data-parallel ranks, ranks 2, 3 repeat the shares of ranks 0, 1
    _, lp_ref, gn_ref, w_ref = step(C(), rank % 2, 4.0)
    for name, ec, share in (("pp2_dp2", C(pipeline_model_parallel_size=2), rank % 2),
                            ("pp2_tp2", C(pipeline_model_parallel_size=2, tensor_model_parallel_size=2), 0)):
        denom = 2.0 if name == "pp2_dp2" else 1.0
        eng, lp, gn, w = step(ec, share, denom)
        assert eng.pp_size == 2 and eng.mp_size == (2 if name == "pp2_dp2" else 4)
        if name == "pp2_dp2":
            torch.testing.assert_close(lp, lp_ref, atol=2e-5, rtol=1e-4)  # every stage reports the last stage's values
            assert abs(gn - gn_ref) < 2e-4 * max(1.0, gn_ref), (name, gn, gn_ref)
            assert set(w) == set(w_ref)
            for k in w_ref:
                d = (w[k] - w_ref[k]).abs()
                assert float(d.max()) <= 2.1e-3 and float(d.mean()) < 2e-5, (name, k, float(d.max()), float(d.mean()))
        else:
            assert torch.isfinite(lp).all() and gn > 0 and set(w) == set(w_ref)
    # the pipelined batch interface: two micro-batches, SFT loss; loss and gradient norm equal the data-parallel run's
    outs = {}
    for name, ec in (("dp", C()), ("pp", C(pipeline_model_parallel_size=2))):
        eng = NativeEngine(cfg, ec, optim, device="cpu", group=dist.group.WORLD, seed=4).initialize()
        seqs = [sample(rank % 2 + 10 * j)[2][:n] for j, n in enumerate((9, 14, 6, 11))]
        nt = lambda xs: torch.nested.as_nested_tensor(xs, layout=torch.jagged)  # noqa: E731
        td = tu.get_tensordict({"input_ids": nt(seqs), "loss_mask": nt([torch.ones_like(s) for s in seqs])},
                               {"temperature": 1.0, "micro_batch_size_per_gpu": 2})
        with eng.train_mode():
            out = eng.train_batch(td, partial(sft_loss_on_batch, None))
        outs[name] = (sum(out["loss"]), out["metrics"]["grad_norm"])
    # the 4-rank data-parallel run holds every sample twice: same global mean, same gradient
    assert abs(outs["dp"][1] - outs["pp"][1]) < 2e-4 * max(1.0, outs["dp"][1]), outs
    dist.barrier()
    if rank == 0:
        print("PP_TRAIN_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
