"""Headline benchmark: end-to-end GRPO step throughput (tokens/s over the whole job) on the
Qwen2.5-7B architecture, random-init weights, synthetic prompts.

    python bench.py --gpus 1 --steps 2 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus 8 --steps 2 --warmup 3

One step = rollout (n samples per prompt, paged-KV engine) -> reward -> old log-probs -> reference log-probs ->
GRPO advantages -> actor update (fwd + bwd + optimizer) -> weight sync to the rollout engine, all through
``RayPPOTrainer.train_step`` in SPMD mode (one controller replica per GPU). Weak scaling: every GPU gets
``--prompts-per-gpu`` prompts (128 prompts x 8 samples at 8 GPUs).

Rank 0 prints one JSON line. The K timed steps are bracketed twice: by CUDA events on the step stream (``value``,
max over ranks) and by the host clock (``e2e``). Every timed step starts from the batch as the data loader hands it
over (host tensors), copies the prompt tensors into pinned host memory and from there to the device, runs
``RayPPOTrainer.train_step`` on those device tensors, and reads the step's loss back to the host.

``--impl reference`` reports whether the unmodified reference can run here; ``--impl stock-libs`` times the same
phases with the libraries the reference is built on (vLLM, HF transformers + torch FSDP2 + flash-attn), none of this
repository's models, kernels or engines on that path (see ``baseline/stock_libs.py``).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

# Tensor-parallel size of a rollout replica when the job has that many GPUs (the benchmark configuration names 2).
DEFAULT_ROLLOUT_TP = 1


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "stock-libs"])
    ap.add_argument("--rollout-tp", type=int, default=0,
                    help="tensor-parallel size of a rollout replica (0 = the benchmark's default: 2 when the job has "
                         "at least 2 GPUs, else 1)")
    ap.add_argument("--breakdown", default="",
                    help="after the timed steps, run update_actor and compute_log_prob once more under the torch "
                         "profiler and write the per-kernel device-time shares to this JSON file (rank 0)")
    ap.add_argument("--phases", default="rollout,logprob,update,resync,fused_ce",
                    help="stock-libs arm: which phases to time")
    ap.add_argument("--config", type=int, default=1, choices=[1, 2],
                    help="1 = GRPO (the headline); 2 = PPO with a critic of the same architecture, GAE, 32 prompts x 1 "
                         "sample per GPU, even-id reward")
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--prompts-per-gpu", type=int, default=None, help="default: 16 (config 1), 32 (config 2)")
    ap.add_argument("--n", type=int, default=None, help="samples per prompt; default: 8 (config 1), 1 (config 2)")
    ap.add_argument("--min-prompt", type=int, default=256)
    ap.add_argument("--max-prompt", type=int, default=512)
    ap.add_argument("--max-response", type=int, default=1024)
    ap.add_argument("--max-token-len", type=int, default=16384)
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (marks the run as reduced)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--agent-loop", action="store_true",
                    help="variant: rollouts through the agent loops and the token-in / token-out server (not the headline path)")
    ap.add_argument("--lora-rank", type=int, default=0, help="variant: LoRA training (not the headline configuration)")
    ap.add_argument("--prefix-sharing", action="store_true",
                    help="variant: the log-prob passes evaluate each prompt once for its n samples (use_prefix_grouper)")
    args = ap.parse_args()
    if args.prompts_per_gpu is None:
        args.prompts_per_gpu = 16 if args.config == 1 else 32
    if args.n is None:
        args.n = 8 if args.config == 1 else 1
    return args


def reference_arm(args):
    """The reference installs only with --no-deps and cannot be imported: ``import verl`` needs ray, tensordict,
    hydra-core, omegaconf, peft, codetiming and accelerate, none of which is installable offline here."""
    ref = os.path.join(REPO, "baseline", "_ref")
    why = None
    if not os.path.isdir(os.path.join(ref, "verl")):
        why = "baseline/_ref is absent: the offline pip install of the reference has not been run in this checkout"
    else:
        probe = subprocess.run([sys.executable, "-c", "import sys; sys.path.insert(0, sys.argv[1]); import verl",
                                ref], capture_output=True, text=True, cwd=tempfile.gettempdir())
        if probe.returncode != 0:
            last = (probe.stderr.strip().splitlines() or ["import failed"])[-1]
            why = f"import verl fails offline ({last}); its dependencies ray/tensordict/hydra-core/omegaconf are not in the wheelhouse"
        else:
            why = "reference imports but its stock main_ppo path needs a Ray cluster and vLLM workers that were not validated here"
    print(json.dumps({"impl": "reference", "unavailable": why}))


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of this process's GPU in the background (read-only queries)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = os.path.join(tempfile.gettempdir(), f"verl_b200_clocks_{os.getpid()}.csv")
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def build_config(args, world: int):
    from verl_b200.utils.config import compose

    per_gpu = args.prompts_per_gpu
    global_prompts = per_gpu * world
    ov = [
        f"actor_rollout_ref.model.path=preset:{args.model}", "trainer.device=cuda", f"trainer.n_gpus_per_node={world}",
        "trainer.nnodes=1", "trainer.logger=[]", "trainer.val_before_train=false", "trainer.save_freq=-1", "trainer.test_freq=-1",
        "trainer.balance_batch=false", "trainer.resume_mode=disable", "trainer.total_epochs=1000",
        f"data.train_files=synthetic:{global_prompts * 4}:{args.min_prompt}:{args.max_prompt}:100:151000:0:synthetic/contains_token:4242",
        "data.val_files=null", f"data.train_batch_size={global_prompts}", f"data.max_prompt_length={args.max_prompt}",
        f"data.max_response_length={args.max_response}", "data.shuffle=false",
        "algorithm.adv_estimator=grpo", f"actor_rollout_ref.rollout.n={args.n}", "actor_rollout_ref.rollout.temperature=1.0",
        f"actor_rollout_ref.rollout.max_num_seqs={max(per_gpu * args.n * args.rollout_tp, 8)}", "actor_rollout_ref.rollout.max_num_batched_tokens=8192",
        f"actor_rollout_ref.rollout.tensor_model_parallel_size={args.rollout_tp}",
        f"actor_rollout_ref.rollout.gpu_memory_utilization={0.12 if args.rollout_tp == 1 else 0.2}",
        "actor_rollout_ref.rollout.log_prob_use_dynamic_bsz=true", f"actor_rollout_ref.rollout.log_prob_max_token_len_per_gpu={2 * args.max_token_len}",
        "actor_rollout_ref.ref.log_prob_use_dynamic_bsz=true", f"actor_rollout_ref.ref.log_prob_max_token_len_per_gpu={2 * args.max_token_len}",
        f"actor_rollout_ref.actor.ppo_mini_batch_size={global_prompts}", "actor_rollout_ref.actor.use_dynamic_bsz=true",
        f"actor_rollout_ref.actor.ppo_max_token_len_per_gpu={args.max_token_len}", "actor_rollout_ref.actor.use_kl_loss=true",
        "actor_rollout_ref.actor.kl_loss_coef=0.001", "actor_rollout_ref.actor.optim.lr=1e-6",
        # the rule-based reward runs on a host thread while the GPUs compute the log-probs (an option of the reference)
        "reward_model.launch_reward_fn_async=true",
    ]
    if args.config == 2:
        # PPO with a critic: GAE (gamma = lambda = 1), value clip 0.5, KL against the reference policy in the reward,
        # reward = fraction of even ids at the last token
        ov = [o for o in ov if not o.startswith(("algorithm.adv_estimator", "data.train_files", "actor_rollout_ref.actor.use_kl_loss"))]
        ov += ["algorithm.adv_estimator=gae", "algorithm.gamma=1.0", "algorithm.lam=1.0",
               "actor_rollout_ref.actor.use_kl_loss=false", "algorithm.use_kl_in_reward=true",
               f"data.train_files=synthetic:{global_prompts * 4}:{args.min_prompt}:{args.max_prompt}:100:151000:0:synthetic/even_fraction",
               f"critic.model.path=preset:{args.model}", "critic.optim.lr=1e-5", "critic.cliprange_value=0.5",
               f"critic.ppo_mini_batch_size={global_prompts}", "critic.use_dynamic_bsz=true",
               f"critic.ppo_max_token_len_per_gpu={args.max_token_len}"]
        if args.layers:
            ov.append(f"+critic.model.override_config.num_hidden_layers={args.layers}")
    if args.layers:
        ov.append(f"+actor_rollout_ref.model.override_config.num_hidden_layers={args.layers}")
    if args.agent_loop:
        ov += ["actor_rollout_ref.rollout.agent.use_agent_loop=true", "actor_rollout_ref.rollout.agent.num_workers=4",
               "data.return_raw_chat=true"]
    if args.prefix_sharing:
        ov.append("actor_rollout_ref.actor.use_prefix_grouper=true")
    if args.lora_rank:
        ov += [f"actor_rollout_ref.model.lora_rank={args.lora_rank}", "actor_rollout_ref.model.lora_alpha=32"]
    return compose("ppo_trainer", ov)


def main():
    args = parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            reference_arm(args)
        return
    if args.impl == "stock-libs":
        from baseline import stock_libs

        stock_libs.main(args)
        return
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl")
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run"
    os.environ["VERL_B200_SPMD"] = "1"
    # the benchmark measures the peer-memory collectives: a failed set-up must abort, not fall back to NCCL
    os.environ["VERL_B200_REQUIRE_PEER_COMM"] = "1"
    if args.rollout_tp <= 0:
        args.rollout_tp = DEFAULT_ROLLOUT_TP if world % DEFAULT_ROLLOUT_TP == 0 else 1
    tp = args.rollout_tp
    assert world % tp == 0, f"--rollout-tp {tp} does not divide {world} GPUs"

    from verl_b200.ops import _lib
    from verl_b200.single_controller.spmd import SPMDResourcePool, SPMDWorkerGroup
    from verl_b200.trainer.main_ppo import build_tokenizer, create_rl_dataset, create_rl_sampler
    from verl_b200.trainer.ppo.ray_trainer import RayPPOTrainer, ResourcePoolManager
    from verl_b200.trainer.ppo.reward import load_reward_manager
    from verl_b200.trainer.ppo.utils import Role
    from verl_b200.workers.engine_workers import ActorRolloutRefWorker

    _lib.load(build_if_missing=False)
    cfg = build_config(args, world)
    tok = build_tokenizer(cfg)
    ds = create_rl_dataset(cfg.data.train_files, cfg.data, tok)
    roles, mapping = {Role.ActorRollout: ActorRolloutRefWorker}, {Role.ActorRollout: "global_pool"}
    if args.config == 2:
        from verl_b200.workers.engine_workers import CriticWorker

        roles[Role.Critic], mapping[Role.Critic] = CriticWorker, "global_pool"
    rpm = ResourcePoolManager({"global_pool": [1]}, mapping, pool_cls=SPMDResourcePool)
    trainer = RayPPOTrainer(config=cfg, tokenizer=tok, role_worker_mapping=roles,
                            resource_pool_manager=rpm, ray_worker_group_cls=SPMDWorkerGroup,
                            reward_fn=load_reward_manager(cfg, tok), val_reward_fn=None, train_dataset=ds,
                            train_sampler=create_rl_sampler(cfg.data, ds), device_name="cuda")
    trainer.init_workers()

    def batches():
        while True:
            for b in trainer.train_dataloader:
                yield b

    it = batches()
    dev = torch.device("cuda", local)
    worker = trainer.actor_rollout_wg.worker.worker_dict["actor_rollout"]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step(batch_dict):
        """The user-facing call. The loader's prompt tensors go to pinned host memory, from there to the device,
        and the step runs on those device tensors; the step's loss is read back to the host."""
        h2d, staged = 0, {}
        for k, v in batch_dict.items():
            if isinstance(v, torch.Tensor):
                pinned = v.pin_memory()
                staged[k] = pinned.to(dev, non_blocking=True)
                h2d += pinned.numel() * pinned.element_size()
            else:
                staged[k] = v
        m = trainer.train_step(staged)
        loss = torch.tensor([m.get("actor/pg_loss", 0.0), m.get("actor/kl_loss", 0.0)], device=dev)
        host = loss.cpu()
        return m, h2d, host.numel() * host.element_size()

    for _ in range(args.warmup):
        step(next(it))

    # ---- timed region: exactly K steps, bracketed by CUDA events (value) and by the host clock (e2e) ----
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    ev0.record()
    tokens, h2d, d2h = 0, 0, 0
    last = {}
    for _ in range(args.steps):
        last, h2d, d2h = step(next(it))
        tokens += int(last["perf/total_num_tokens"])
    ev1.record()
    barrier()
    host_s = time.perf_counter() - t0
    red = torch.tensor([ev0.elapsed_time(ev1), host_s * 1e3], device=dev)
    launches = torch.tensor([float(_lib.launch_count() - launches0)], device=dev)
    if world > 1:
        dist.all_reduce(red, op=dist.ReduceOp.MAX)
        dist.all_reduce(launches)
    clocks = sampler.stop() if rank == 0 else {}
    total_ms, host_ms = red.tolist()
    e2e = None
    if not args.no_e2e:
        # the data loader yields the global batch on every rank: each rank stages all of it, as a user's loop would
        e2e = {"value": tokens / (host_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d) * world,
               "d2h_bytes_per_step": int(d2h) * world,
               "timer": "host clock around the same K steps (max over ranks), each step: loader batch -> pinned host -> "
                        "device -> train_step on the device tensors -> loss read back"}
    comm = getattr(worker, "comm_kind", "none")
    # the last step's rollout times of every rank (a straggler shows here, not in rank 0's breakdown)
    rt = getattr(worker, "last_rollout_times", {})
    mine = torch.tensor([rt.get("generate_s", 0.0), rt.get("sleep_s", 0.0), rt.get("engine_step_s", 0.0)], device=dev)
    per_rank = [torch.zeros_like(mine) for _ in range(world)]
    if world > 1:
        dist.all_gather(per_rank, mine)
    else:
        per_rank = [mine]
    per_rank = [[round(float(x), 3) for x in t.tolist()] for t in per_rank]

    if rank == 0:
        c = worker.model_config
        out = {
            "metric": ("RL step tokens/s/box (GRPO, rollout+logprob+ref+update+resync)" if args.config == 1 else
                       "RL step tokens/s/box (PPO + critic, rollout+logprob+values+update_critic+update_actor+resync)"),
            "value": tokens / (total_ms / 1e3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic prompts (uniform ids), random-init weights", "impl": "ours",
            "config": {"model": (args.model if not args.layers else f"{args.model}-REDUCED-{args.layers}L")
                       + ("+agent-loop-rollout" if args.agent_loop else "") + (f"+lora{args.lora_rank}" if args.lora_rank else "") + ("+prefix-sharing-logprob" if args.prefix_sharing else ""),
                       "benchmark_config": args.config, "layers": c.num_hidden_layers, "hidden": c.hidden_size, "vocab": c.vocab_size,
                       "global_batch": args.prompts_per_gpu * world * args.n, "prompts": args.prompts_per_gpu * world,
                       "n_samples": args.n, "seq_len": args.max_prompt + args.max_response,
                       "prompt_len": [args.min_prompt, args.max_prompt], "max_response": args.max_response,
                       "parallelism": f"zero3-dp{world}, rollout tp{tp} x {world // tp} replicas", "rollout_tp": tp,
                       "comm": comm, "nvls": bool(getattr(getattr(worker, "comm", None), "use_nvls", False)),
                       "cache": "inputs larger than L2 (15 GB of weights streamed per pass)",
                       "timer": "CUDA events on the step stream, max over ranks"},
            "clocks": clocks, "gpu_launches": int(launches.item()),
            "breakdown_s": {k.split("/", 1)[1]: round(v, 3) for k, v in last.items() if k.startswith("timing_s/")},
            "rollout_tokens_per_s_per_gpu": last.get("rollout/tokens_per_s"),
            "rollout_engine": {k.split("engine_", 1)[1]: round(v, 3) for k, v in last.items() if k.startswith("rollout/engine_")},
            "rollout_per_rank": {"columns": ["generate_s", "sleep_s", "engine_step_s"], "rows": per_rank},
            "resync_ms": 1e3 * last.get("timing_s/resync", 0.0),
            "mfu_actor": last.get("perf/mfu/actor"),
            "kept_activation_layers": getattr(worker.actor_engine, "last_kept_layers", 0),
            "peak_mem_gb": {"allocated": round(torch.cuda.max_memory_allocated() / 2**30, 1),
                            "reserved": round(torch.cuda.max_memory_reserved() / 2**30, 1)},
            "keep_info": getattr(worker.actor_engine, "last_keep_info", None),
        }
        if e2e is not None:
            out["e2e"] = e2e
        print(json.dumps(out))
    if args.breakdown:
        from verl_b200.utils.profiler.kernel_breakdown import kernel_breakdown

        b = trainer._last_batch
        # with programmatic dependent launch a kernel's recorded duration includes its wait for the kernel before it;
        # the breakdown pass runs in plain stream order so that per-kernel times add up
        _lib.set_pdl(False)
        res = {"n_gpus": world, "note": "device times under the torch profiler: shares only; plain stream order"}
        res["update_actor"] = kernel_breakdown(lambda: trainer.actor_rollout_wg.update_actor(b))
        res["compute_log_prob"] = kernel_breakdown(lambda: trainer.actor_rollout_wg.compute_log_prob(b))
        if rank == 0:
            with open(args.breakdown, "w") as f:
                json.dump(res, f, indent=1)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
