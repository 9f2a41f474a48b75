"""Same-box yardstick built from the libraries the reference runs on (``bench.py --impl stock-libs``).

The unmodified reference cannot be imported offline (no ray / tensordict / hydra), so its GRPO step is timed phase by
phase with the libraries it delegates to, on the benchmark's shapes (Qwen2.5-7B architecture, random weights, 16 prompts
x 8 samples per GPU, prompts of 256-512 tokens, responses of up to 1024 tokens):

* ``rollout``  vLLM ``LLM.generate`` on token-id prompts (what verl/workers/rollout/vllm_rollout drives), one replica per
  ``--rollout-tp`` GPUs;
* ``logprob``  HF ``Qwen2ForCausalLM`` under torch FSDP2 with flash-attn varlen on packed micro-batches and full logits
  (verl/workers/actor/dp_actor.py:_forward_micro_batch with ``use_remove_padding``), no gradients;
* ``update``   the same model: forward + backward with gradient checkpointing, PPO-clip + low-variance KL loss, gradient
  clipping, ``torch.optim.AdamW`` (verl/workers/actor/dp_actor.py:update_policy);
* ``resync``   the reference's weight-sync algorithm (verl/workers/fsdp_workers.py:677-756): per parameter
  ``full_tensor()`` (NCCL all-gather), copy into a 2 GB bucket, copy out into the inference engine's tensors;
* ``fused_ce`` the reference's own Triton linear-cross-entropy kernel (``verl/utils/kernel/kernels.py``, loaded from the
  installed reference by file path, source untouched), forward and forward + backward at T = 16384, V = 152064.

Nothing of this repository's package is imported here. Every phase runs in a process of its own (vLLM wants one) and
prints one JSON line; the parent merges them into one line with ``"impl": "stock-libs"``.
"""

from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))

QWEN25_7B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=152064, hidden_size=3584,
                 intermediate_size=18944, num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4,
                 rope_theta=1e6, max_position_embeddings=32768, rms_norm_eps=1e-6, tie_word_embeddings=False,
                 hidden_act="silu", torch_dtype="bfloat16", bos_token_id=151643, eos_token_id=151645, use_cache=True,
                 attention_dropout=0.0, initializer_range=0.02, use_sliding_window=False)


def _prompts(n_prompts: int, lo: int, hi: int, seed: int):
    import random

    rnd = random.Random(seed)
    return [[rnd.randrange(100, 151000) for _ in range(rnd.randint(lo, hi))] for _ in range(n_prompts)]


# --------------------------------------------------------------------------------------------------- rollout (vLLM)
def phase_rollout(a) -> dict:
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
    os.environ.setdefault("VLLM_NO_USAGE_STATS", "1")
    os.environ.setdefault("VLLM_WORKER_MULTIPROC_METHOD", "spawn")
    d = tempfile.mkdtemp(prefix="stock_qwen7b_")
    cfg = dict(QWEN25_7B)
    if a["layers"]:
        cfg["num_hidden_layers"] = a["layers"]
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    from vllm import LLM, SamplingParams

    tp, n = a["tp"], a["n"]
    n_prompts = a["prompts_per_gpu"] * tp
    t0 = time.perf_counter()
    llm = LLM(model=d, skip_tokenizer_init=True, load_format="dummy", dtype="bfloat16", tensor_parallel_size=tp,
              gpu_memory_utilization=0.5, max_model_len=a["max_prompt"] + a["max_response"],
              max_num_seqs=n_prompts * n, max_num_batched_tokens=8192, enable_prefix_caching=True, seed=0,
              generation_config="vllm", disable_log_stats=True)
    init_s = time.perf_counter() - t0
    sp = SamplingParams(temperature=1.0, top_p=1.0, top_k=-1, max_tokens=a["max_response"], logprobs=0, detokenize=False)

    def run(seed):
        reqs = [{"prompt_token_ids": p} for p in _prompts(n_prompts, a["min_prompt"], a["max_prompt"], seed)
                for _ in range(n)]
        t = time.perf_counter()
        outs = llm.generate(reqs, sp, use_tqdm=False)
        dt = time.perf_counter() - t
        return dt, sum(len(o.outputs[0].token_ids) for o in outs), sum(len(r["prompt_token_ids"]) for r in reqs)

    run(100)  # warm-up: graphs captured, caches allocated; different prompts, so the prefix cache does not hit later
    times = [run(s) for s in range(a["repeats"])]
    dt, gen, prm = min(times)
    import vllm

    return {"phase": "rollout", "lib": f"vllm {vllm.__version__}", "tp": tp, "seqs": n_prompts * n, "gen_s": dt,
            "response_tokens": gen, "prompt_tokens": prm, "tokens_per_s_per_gpu": gen / dt / tp,
            "all_runs_s": [round(t[0], 3) for t in times], "engine_init_s": round(init_s, 1)}


# ------------------------------------------------------------------------------------- HF + FSDP2 + flash-attn phases
def _build_fsdp_model(a, trainable: bool):
    import torch
    import torch.distributed as dist
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
    from transformers import AutoModelForCausalLM, Qwen2Config

    cfg = {k: v for k, v in QWEN25_7B.items() if k not in ("architectures", "torch_dtype", "model_type")}
    if a["layers"]:
        cfg["num_hidden_layers"] = a["layers"]
    hf_cfg = Qwen2Config(**cfg)
    torch.manual_seed(0)
    # the reference keeps the actor's parameters in fp32 and computes in bf16 (fsdp_workers.py: mixed precision
    # param_dtype=bf16, reduce_dtype=fp32) with flash-attn on packed inputs
    with torch.device("cuda"):
        model = AutoModelForCausalLM.from_config(hf_cfg, attn_implementation="flash_attention_2", dtype=torch.float32)
    model.config.use_cache = False
    if trainable:
        model.gradient_checkpointing_enable(gradient_checkpointing_kwargs={"use_reentrant": False})
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    mesh = dist.device_mesh.init_device_mesh("cuda", (dist.get_world_size(),))
    for layer in model.model.layers:
        fully_shard(layer, mesh=mesh, mp_policy=mp)
    fully_shard(model, mesh=mesh, mp_policy=mp)
    return model


def _micro_batches(seqs, budget):
    out, cur, tok = [], [], 0
    for s in seqs:
        if cur and tok + len(s) > budget:
            out.append(cur)
            cur, tok = [], 0
        cur.append(s)
        tok += len(s)
    if cur:
        out.append(cur)
    return out


def _pack(mb, dev):
    import torch

    ids = torch.tensor([t for s in mb for t in s], device=dev).unsqueeze(0)
    pos = torch.cat([torch.arange(len(s), device=dev) for s in mb]).unsqueeze(0)
    return ids, pos


def _logprob_entropy(logits, labels, temperature=1.0, entropy=True):
    """Full-logit path of verl/utils/torch_functional.py (logprobs_from_logits / entropy_from_logits)."""
    import torch

    logits = logits.float() / temperature
    lse = torch.logsumexp(logits, dim=-1)
    lp = logits.gather(-1, labels.unsqueeze(-1)).squeeze(-1) - lse
    ent = None
    if entropy:
        ent = lse - (torch.softmax(logits, dim=-1) * logits).sum(-1)
    return lp, ent


def phase_train(a) -> dict:
    import torch
    import torch.distributed as dist

    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29577")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    model = _build_fsdp_model(a, trainable=True)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-6, betas=(0.9, 0.999), weight_decay=0.01)
    n_seq = a["prompts_per_gpu"] * a["n"]
    import random

    rnd = random.Random(1000 + rank)
    seqs = [[rnd.randrange(100, 151000) for _ in range(rnd.randint(a["min_prompt"], a["max_prompt"]) + a["max_response"])]
            for _ in range(n_seq)]
    tokens = sum(len(s) for s in seqs)
    out = {"phase": "train", "lib": f"transformers + torch FSDP2 + flash_attn, torch {torch.__version__}", "world": world,
           "seqs_per_gpu": n_seq, "tokens_per_gpu": tokens}

    def timed(fn, reps):
        best = None
        for _ in range(reps):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / 1e3], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            best = t.item() if best is None else min(best, t.item())
        return best

    def log_prob(budget):
        model.eval()
        with torch.no_grad():
            for mb in _micro_batches(seqs, budget):
                ids, pos = _pack(mb, dev)
                logits = model(input_ids=ids, position_ids=pos, use_cache=False).logits.squeeze(0)
                _logprob_entropy(logits[:-1], ids[0, 1:], entropy=True)

    def update(budget):
        model.train()
        opt.zero_grad(set_to_none=True)
        mbs = _micro_batches(seqs, budget)
        for mb in mbs:
            ids, pos = _pack(mb, dev)
            logits = model(input_ids=ids, position_ids=pos, use_cache=False).logits.squeeze(0)
            lp, _ = _logprob_entropy(logits[:-1], ids[0, 1:], entropy=False)
            old, ref = lp.detach() + 0.01, lp.detach() - 0.01
            adv = torch.ones_like(lp)
            ratio = torch.exp(lp - old)
            pg = torch.max(-adv * ratio, -adv * ratio.clamp(0.8, 1.2)).mean()
            kl = ref - lp
            klv = (torch.exp(kl) - kl - 1).clamp(-10, 10).mean()
            ((pg + 0.001 * klv) / len(mbs)).backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()

    for name, fn, budget in (("old_log_prob_s", log_prob, 2 * a["max_token_len"]), ("update_actor_s", update, a["max_token_len"])):
        b = budget
        while True:
            try:
                fn(b)  # warm-up
                out[name] = timed(lambda: fn(b), a["repeats"])
                out[name.replace("_s", "_token_budget")] = b
                break
            except torch.OutOfMemoryError:
                torch.cuda.empty_cache()
                b //= 2
                if b < 2048:
                    out[name] = None
                    out[name.replace("_s", "_error")] = "out of memory down to a 2048-token micro-batch"
                    break
    out["peak_mem_gb"] = round(torch.cuda.max_memory_allocated() / 2**30, 1)

    # ---- the reference's weight-sync algorithm on this sharded model ----
    if "resync" in a["phases"]:
        from torch.distributed.tensor import DTensor

        dest = {n: torch.empty(p.shape, dtype=torch.bfloat16, device=dev) for n, p in model.named_parameters()}
        bucket = torch.empty(min(2 << 30, 2 * sum(v.numel() for v in dest.values())), dtype=torch.uint8, device=dev)

        def resync():
            off, pending = 0, []
            with torch.no_grad():
                for n, p in model.named_parameters():
                    full = p.full_tensor() if isinstance(p, DTensor) else p
                    full = full.to(torch.bfloat16)
                    nb = full.numel() * 2
                    if off + nb > bucket.numel():
                        for dn, o, m in pending:  # receiver side: copy out of the bucket into the engine's tensors
                            dest[dn].view(-1).view(torch.uint8).copy_(bucket[o : o + m])
                        off, pending = 0, []
                    bucket[off : off + nb].copy_(full.reshape(-1).view(torch.uint8))
                    pending.append((n, off, nb))
                    off += nb
                for dn, o, m in pending:
                    dest[dn].view(-1).view(torch.uint8).copy_(bucket[o : o + m])

        resync()
        out["resync_ms"] = 1e3 * timed(resync, a["repeats"])
        out["resync_gb"] = round(sum(v.numel() for v in dest.values()) * 2 / 1e9, 2)
    dist.barrier()
    return out


# ------------------------------------------------------------------------------- the reference's Triton fused CE kernel
def _load_reference_kernels():
    """``verl.utils.kernel.{kernels,linear_cross_entropy}`` and ``verl.utils.device`` from the installed reference,
    by file path: ``import verl`` itself needs ray and friends, the three files need only torch and triton."""
    import importlib.util
    import types

    ref = os.path.join(HERE, "_ref", "verl")
    for name in ("verl", "verl.utils", "verl.utils.kernel"):
        mod = types.ModuleType(name)
        mod.__path__ = [os.path.join(ref, *name.split(".")[1:])]
        sys.modules[name] = mod
    for name in ("verl.utils.device", "verl.utils.kernel.kernels", "verl.utils.kernel.linear_cross_entropy"):
        path = os.path.join(ref, *name.split(".")[1:]) + ".py"
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
    return sys.modules["verl.utils.kernel.linear_cross_entropy"].linear_cross_entropy


def phase_fused_ce(a) -> dict:
    import torch

    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    lce = _load_reference_kernels()
    T, H, V = a["ce_tokens"], 3584, 152064
    g = torch.Generator(device="cuda").manual_seed(0)
    hidden = (torch.randn(T, H, device="cuda", generator=g) * 1.0).to(torch.bfloat16).requires_grad_(True)
    weight = (torch.randn(V, H, device="cuda", generator=g) * 0.02).to(torch.bfloat16).requires_grad_(True)
    labels = torch.randint(0, V, (T,), device="cuda", generator=g)

    def fwd():
        with torch.no_grad():
            return lce(hidden, weight, labels, 1.0, "none")

    g_lp = torch.rand(T, device="cuda", generator=g)
    g_ent = torch.zeros(T, device="cuda")

    def fwd_bwd():
        hidden.grad = weight.grad = None
        lp, ent = lce(hidden, weight, labels, 1.0, "none")
        torch.autograd.backward([lp, ent], [g_lp, g_ent])

    def timed(fn, reps=5):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(reps):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return min(ts)

    f = timed(fwd)
    fb = timed(fwd_bwd)
    fl = 2.0 * T * H * V
    import triton

    return {"phase": "fused_ce", "lib": f"reference Triton kernel (triton {triton.__version__})", "T": T, "H": H, "V": V,
            "fwd_ms": f, "fwd_tflops": fl / f / 1e9, "fwd_bwd_ms": fb, "fwd_bwd_tflops": 3 * fl / fb / 1e9}


PHASES = {"rollout": phase_rollout, "train": phase_train, "fused_ce": phase_fused_ce}


def _child(phase: str, a: dict, env: dict, timeout: int):
    """Run one phase in a fresh interpreter (cwd outside the repository, so that nothing of it is importable)."""
    cmd = [sys.executable, os.path.abspath(__file__), "--child", phase, json.dumps(a)]
    try:
        res = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=tempfile.gettempdir(), timeout=timeout)
    except subprocess.TimeoutExpired:
        return {"phase": phase, "error": f"no result within {timeout} s"}
    for line in reversed(res.stdout.strip().splitlines()):
        if line.startswith("{\"phase\""):
            return json.loads(line)
    tail = (res.stderr.strip().splitlines() or ["no output"])[-6:]
    return {"phase": phase, "error": " | ".join(t[-300:] for t in tail)}


def main(args) -> None:
    """Entry from ``bench.py --impl stock-libs``: under ``torch.distributed.run`` every rank runs the training phases,
    one rank per rollout replica runs vLLM on the replica's GPUs, rank 0 prints the merged line."""
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    sync = None
    if world > 1:  # host-side barrier between the phases: a replica's vLLM run must not share its GPUs with the next phase
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo")
        sync = dist.barrier
    tp = args.rollout_tp if args.rollout_tp > 0 else 1
    phases = [p.strip() for p in args.phases.split(",") if p.strip()]
    a = dict(layers=args.layers, tp=tp, n=args.n, prompts_per_gpu=args.prompts_per_gpu, min_prompt=args.min_prompt,
             max_prompt=args.max_prompt, max_response=args.max_response, max_token_len=args.max_token_len,
             repeats=max(1, min(args.steps, 3)), phases=phases, ce_tokens=16384)
    results = {}
    base_env = {k: v for k, v in os.environ.items()
                if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT", "LOCAL_WORLD_SIZE",
                             "GROUP_RANK", "ROLE_RANK", "ROLE_WORLD_SIZE", "TORCHELASTIC_RUN_ID", "GROUP_WORLD_SIZE",
                             "ROLE_NAME", "TORCHELASTIC_RESTART_COUNT", "TORCHELASTIC_MAX_RESTARTS",
                             "TORCHELASTIC_USE_AGENT_STORE", "TORCH_NCCL_ASYNC_ERROR_HANDLING", "TORCHELASTIC_ERROR_FILE")}
    base_env["PYTHONPATH"] = ""
    if "rollout" in phases and local % tp == 0 and local + tp <= world:
        env = dict(base_env)
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        ids = vis.split(",") if vis else [str(i) for i in range(world)]
        env["CUDA_VISIBLE_DEVICES"] = ",".join(ids[local : local + tp])
        results["rollout"] = _child("rollout", a, env, timeout=900)
    if sync is not None:
        sync()
    if any(p in phases for p in ("logprob", "update", "resync")):
        env = dict(base_env)
        env.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(local), "MASTER_ADDR": "127.0.0.1",
                    "MASTER_PORT": str(int(os.environ.get("MASTER_PORT", "29500")) + 7)})
        results["train"] = _child("train", a, env, timeout=900)
    if "fused_ce" in phases and rank == 0:
        env = dict(base_env)
        env["LOCAL_RANK"] = str(local)
        results["fused_ce"] = _child("fused_ce", a, env, timeout=600)
    if sync is not None:
        sync()
    if rank != 0:
        return
    ro, tr = results.get("rollout", {}), results.get("train", {})
    line = {"impl": "stock-libs", "metric": "GRPO step phases with vLLM / HF transformers + torch FSDP2 + flash-attn",
            "n_gpus": world, "dtype": "bf16", "data": "synthetic prompts (uniform ids), random-init weights",
            "config": {"model": "qwen2.5-7b" + (f"-REDUCED-{args.layers}L" if args.layers else ""), "rollout_tp": tp,
                       "prompts_per_gpu": args.prompts_per_gpu, "n_samples": args.n,
                       "prompt_len": [args.min_prompt, args.max_prompt], "max_response": args.max_response},
            "phases": results}
    gen, lp, up = ro.get("gen_s"), tr.get("old_log_prob_s"), tr.get("update_actor_s")
    if gen and lp and up:
        step = gen + 2 * lp + up + (tr.get("resync_ms") or 0.0) / 1e3
        tok = tr["tokens_per_gpu"] * world
        line.update({"value": tok / step, "unit": "tokens/s", "higher_is_better": True,
                     "composition": "tokens / (gen + 2 x log_prob (actor, reference) + update_actor + resync); phases "
                                    "timed separately, so nothing of a trainer's glue is included"})
    print(json.dumps(line))


if __name__ == "__main__":
    if len(sys.argv) >= 4 and sys.argv[1] == "--child":
        res = PHASES[sys.argv[2]](json.loads(sys.argv[3]))
        print(json.dumps(res), flush=True)
