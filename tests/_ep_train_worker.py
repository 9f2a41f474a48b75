"""Child of tests/test_ep_training_on_cpu.py: 2 gloo ranks. Training an MoE model with expert_model_parallel_size = 2
(every rank owns half of the experts, tokens travel by all-to-all, the expert matrices are never gathered) gives the
log-probs, gradient norm and updated weights of plain ZeRO-3 training (all experts gathered on every rank)."""
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

    cfg = preset("tiny-qwen3-moe")
    optim = C(lr=1e-3, weight_decay=0.01, clip_grad=1.0)
    lens = [9, 14, 6]
    ids = torch.randint(0, cfg.vocab_size, (sum(lens),), generator=torch.Generator().manual_seed(7 + rank))
    batch = PackedBatch(ids, torch.cat([torch.arange(n) for n in lens]), torch.tensor([0, 9, 23, 29], dtype=torch.int32), 14)
    rows, labels = torch.arange(ids.numel()), torch.roll(ids, -1)
    res = {}
    for ep in (1, 2):
        eng = NativeEngine(cfg, C(expert_model_parallel_size=ep), optim, device="cpu", group=dist.group.WORLD, seed=4).initialize()
        if ep == 2:
            mlp = eng.model.layers[0].mlp
            assert mlp.gate_up_proj.shape[0] == cfg.num_experts // 2 and sum(u.local for u in eng.zero.units) == 2 * cfg.num_hidden_layers
        with eng.train_mode():
            eng.optimizer_zero_grad()
            for _ in range(2):  # two micro-batches
                lp, ent = eng.forward_logprob(batch, rows, labels, 1.0)
                ((-lp.mean() + 0.01 * ent.mean()) / 4).backward()
            gn = float(eng.optimizer_step())
        res[ep] = (lp.detach().clone(), gn, {k: v.float().clone() for k, v in eng.zero.named_full_tensors()})
        if ep == 2:
            eng.save_checkpoint(os.path.join(out_dir, "ep"))
    torch.testing.assert_close(res[2][0], res[1][0], atol=2e-5, rtol=1e-4)
    assert abs(res[1][1] - res[2][1]) < 2e-4 * max(1.0, res[1][1]), (res[1][1], res[2][1])
    for k, v in res[1][2].items():
        d = (v - res[2][2][k]).abs()
        assert v.shape == res[2][2][k].shape and float(d.max()) <= 2.1e-3 and float(d.mean()) < 2e-5, (k, float(d.max()))
    # the checkpoint of the expert-parallel engine restores a plain one (same flat shards on disk)
    eng = NativeEngine(cfg, C(), optim, device="cpu", group=dist.group.WORLD, seed=77).initialize()
    eng.load_checkpoint(os.path.join(out_dir, "ep"), load_contents=("model",))
    for k, v in eng.zero.named_full_tensors():
        torch.testing.assert_close(v.float(), res[2][2][k], atol=1e-6, rtol=1e-5)
    if rank == 0:
        print("EP_TRAIN_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
