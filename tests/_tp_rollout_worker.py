"""Child of the tensor-parallel rollout tests (2 ranks; gloo on CPU, NCCL + peer memory on CUDA): a replica whose
weights are sliced over the ranks generates the same greedy tokens as the whole model on one rank, with log-probs that
agree, for a dense model, a model with fewer KV heads than ranks, and expert-parallel MoE layers."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    use_cuda = sys.argv[1] == "cuda"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if use_cuda:
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", device_id=dev)
        from verl_b200.parallel.peer_comm import PeerComm

        comm = PeerComm(dist.group.WORLD)
        dtype, lp_tol = torch.bfloat16, 6e-2
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
        comm, dtype, lp_tol = None, torch.float32, 1e-4
    from verl_b200.models import CausalLM, preset
    from verl_b200.parallel.reshard import shard_state_dict, tp_model_config
    from verl_b200.rollout import NativeRolloutEngine, SamplingParams

    cases = {
        "dense": preset("tiny-qwen2", hidden_size=256, num_attention_heads=2, num_key_value_heads=2, head_dim=128,
                        intermediate_size=512) if use_cuda else preset("tiny-qwen2"),
        "kv_replicated": preset("tiny-qwen2", hidden_size=256, num_attention_heads=2, num_key_value_heads=1, head_dim=128,
                                intermediate_size=512) if use_cuda else preset("tiny-qwen2", num_key_value_heads=1),
        "moe": preset("tiny-qwen3-moe", num_attention_heads=2, num_key_value_heads=2, head_dim=128) if use_cuda
        else preset("tiny-qwen3-moe"),
    }
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, 2000, (n,), generator=g).tolist() for n in (9, 17, 5, 12, 20, 7)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    for name, cfg in cases.items():
        full = CausalLM(cfg, dtype=dtype, device=dev).init_weights(11)
        kw = dict(max_num_seqs=8, max_model_len=64, max_num_batched_tokens=64, num_blocks=64, seed=5)
        ref = NativeRolloutEngine(full, **kw).generate(prompts, sp)
        tp_cfg = tp_model_config(cfg, rank, world)
        part = CausalLM(tp_cfg, dtype=dtype, device=dev)
        part.load_state_dict(shard_state_dict(cfg, dict(full.state_dict()), rank, world), strict=True)
        eng = NativeRolloutEngine(part, tp_group=dist.group.WORLD, tp_comm=comm, full_config=cfg, **kw)
        out = eng.generate(prompts, sp)
        # a second round reuses the engine (graphs captured, buffers alternate) and samples: ranks must stay in lockstep
        out2 = eng.generate(prompts, SamplingParams(temperature=1.0, max_tokens=12, ignore_eos=True))
        toks = torch.tensor([o.token_ids for o in out2], device=dev)
        both = [torch.empty_like(toks) for _ in range(world)]
        dist.all_gather(both, toks)
        assert all(torch.equal(b, both[0]) for b in both), f"{name}: sampled tokens differ between the ranks of a replica"
        n_same = 0
        for a, b in zip(ref, out):
            same = a.token_ids == b.token_ids
            n_same += int(same)
            k = next((i for i, (x, y) in enumerate(zip(a.token_ids, b.token_ids)) if x != y), len(a.token_ids))
            if k:  # log-probs agree up to the first differing token (bf16: near-ties may flip an argmax)
                d = (torch.tensor(a.log_probs[:k]) - torch.tensor(b.log_probs[:k])).abs().max().item()
                assert d < lp_tol, (name, d)
            if not use_cuda:
                assert same, (name, a.token_ids, b.token_ids)
        assert n_same >= len(prompts) - 1, (name, n_same)
        if comm is not None:
            comm.check()
        del eng, ref
    dist.barrier()
    if rank == 0:
        print("TP_ROLLOUT_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
