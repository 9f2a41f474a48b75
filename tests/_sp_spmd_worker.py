"""Child of tests/test_ulysses_on_cpu.py::test_update_policy_with_sp_matches_dp (and, with the argument ``cp``, of
tests/test_context_parallel.py): 2 gloo ranks under an SPMD launch.
``update_actor`` with ulysses_sequence_parallel_size=2 (or context_parallel_size=2) (the two ranks pool their shares and work on the same samples)
must give the loss, gradient norm, number of optimizer steps and weights of a run without sequence parallelism in which
the ranks train on their own shares (data parallel)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    os.environ["VERL_B200_SPMD"] = "1"
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    from verl_b200 import DataProto
    from verl_b200.utils.config import compose
    from verl_b200.workers.engine_workers import ActorRolloutRefWorker

    key = {"sp": "ulysses_sequence_parallel_size", "cp": "context_parallel_size"}[sys.argv[1] if len(sys.argv) > 1 else "sp"]

    def build(sp):
        cfg = compose("ppo_trainer", [
            "actor_rollout_ref.model.path=preset:tiny-qwen2", "trainer.device=cpu", "actor_rollout_ref.rollout.n=1",
            "actor_rollout_ref.rollout.tensor_model_parallel_size=1",
            "actor_rollout_ref.actor.ppo_mini_batch_size=8", "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=2",
            "actor_rollout_ref.actor.use_kl_loss=false", "actor_rollout_ref.actor.optim.lr=1e-3",
            f"actor_rollout_ref.actor.fsdp_config.{key}={sp}",
            "actor_rollout_ref.rollout.max_num_seqs=8", "actor_rollout_ref.rollout.max_num_batched_tokens=64",
            "data.max_prompt_length=8", "data.max_response_length=8"])
        w = ActorRolloutRefWorker(cfg.actor_rollout_ref, role="actor", device_name="cpu")
        w.init_model()
        return w

    def share(r):
        g = torch.Generator().manual_seed(100 + r)
        B, P, R = 4, 8, 8
        ids = torch.randint(3, 2000, (B, P + R), generator=g)
        mask = torch.ones(B, P + R, dtype=torch.long)
        mask[0, :3] = 0
        mask[1, -2:] = 0
        pos = (mask.cumsum(-1) - 1).clamp(min=0)
        return DataProto.from_dict({"input_ids": ids, "attention_mask": mask, "position_ids": pos, "responses": ids[:, P:],
                                    "response_mask": mask[:, P:], "old_log_probs": -torch.rand(B, R, generator=g),
                                    "advantages": torch.randn(B, R, generator=g)}, meta_info={"temperature": 1.0})

    res = {}
    for sp in (1, 2):
        w = build(sp)
        out = w.update_actor(share(rank))
        m = out.meta_info["metrics"]
        res[sp] = (m["actor/pg_loss"], m["actor/grad_norm"], w.actor_engine.zero.master.clone())
    # global mini-batch 8: data parallel = one step over rank 0's and rank 1's four samples; sp = 2 = one step over the
    # pooled eight samples. Same samples, same global token-mean: same loss, gradient norm and weights.
    (l1, g1, w1), (l2, g2, w2) = res[1], res[2]
    assert len(g1) == len(g2) == 1, (len(g1), len(g2))
    t = torch.tensor([l1[0]], dtype=torch.float64)
    dist.all_reduce(t)  # data parallel: a rank reports its own samples' part of the global mean
    assert abs(t.item() - l2[0]) < 1e-5 and abs(g1[0] - g2[0]) < 1e-4 * max(1.0, g1[0]), (t.item(), l2, g1, g2)
    d = (w1 - w2).abs()  # AdamW normalises the step: where a gradient is next to zero, rounding may move a whole lr
    assert float((d > 2e-6).float().mean()) < 1e-3 and float(d.max()) <= 2.1e-3, (float(d.max()),)
    if rank == 0:
        print("SP_SPMD_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
