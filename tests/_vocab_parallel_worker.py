"""Child of tests/test_compat_modules_on_cpu.py: 2 gloo ranks, each holding half of the vocabulary of some logits."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    dist.init_process_group("gloo")
    rank, tp = dist.get_rank(), dist.get_world_size()
    from verl_b200.parallel.vocab_parallel import (vocab_parallel_entropy, vocab_parallel_log_probs_from_logits,
                                                   vocab_parallel_log_probs_from_logits_response_rmpad)

    g = torch.Generator().manual_seed(3)
    B, S, V, R = 3, 7, 24, 4
    full = (torch.randn(B, S, V, generator=g) * 3).requires_grad_(True)
    labels = torch.randint(0, V, (B, S), generator=g)
    w_lp, w_ent = torch.randn(B, S, generator=g), torch.randn(B, S, generator=g)
    ref_ls = torch.log_softmax(full, -1)
    ref_lp = ref_ls.gather(-1, labels[..., None])[..., 0]
    ref_ent = -(ref_ls.exp() * ref_ls).sum(-1)
    ((ref_lp * w_lp).sum() + (ref_ent * w_ent).sum()).backward()
    vs = V // tp
    shard = full.detach()[..., rank * vs:(rank + 1) * vs].clone().requires_grad_(True)
    lp = vocab_parallel_log_probs_from_logits(shard, labels, dist.group.WORLD)
    ent = vocab_parallel_entropy(shard, dist.group.WORLD)
    torch.testing.assert_close(lp, ref_lp.detach(), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(ent, ref_ent.detach(), atol=1e-5, rtol=1e-5)
    ((lp * w_lp).sum() + (ent * w_ent).sum()).backward()
    torch.testing.assert_close(shard.grad, full.grad[..., rank * vs:(rank + 1) * vs], atol=1e-5, rtol=1e-5)

    # packed variant: left-padded prompts, logits of the kept positions only
    mask = torch.ones(B, S, dtype=torch.long)
    mask[0, :2] = 0
    mask[2, :1] = 0
    ids = torch.randint(0, V, (B, S), generator=g)
    rm = shard.detach().reshape(B * S, vs)[mask.bool().reshape(-1)]
    out = vocab_parallel_log_probs_from_logits_response_rmpad(ids, mask, rm, R, dist.group.WORLD)
    want = ref_ls.detach()[:, :-1].gather(-1, ids[:, 1:, None])[..., 0][:, -R:]
    torch.testing.assert_close(out, want, atol=1e-5, rtol=1e-5)
    dist.barrier()
    if rank == 0:
        print("VOCAB_PARALLEL_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
