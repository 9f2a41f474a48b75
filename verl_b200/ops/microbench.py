"""Kernel micro-benchmarks (one kernel per invocation, CUDA-event timing, inputs larger than L2 or rotated).

    python -m verl_b200.ops.microbench gemm --m 8192 --n 8192 --k 8192
    python -m verl_b200.ops.microbench gemm --m 128 --n 3584 --k 18944          # split-K path
    python -m verl_b200.ops.microbench lmhead --t 8192
    python -m verl_b200.ops.microbench decode --batch 128 --ctx 900
    python -m verl_b200.ops.microbench decode_step --batch 128 --layers 4
    python -m verl_b200.ops.microbench attn --batch 16 --ctx 1024 --library

Every run prints one JSON line with the time per call, the achieved rate and (``--library``) the same
measurement for the library kernel (cuBLAS through torch.matmul) as a yardstick. ``--iters 1 --warmup 1``
keeps a profiler capture short.
"""

from __future__ import annotations

import argparse
import json

import torch


def _time(fn, iters: int, warmup: int, graph: bool = True) -> float:
    """Microseconds per call. With ``graph`` the calls are captured once so that host overhead is not timed."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph and iters > 1:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                fn()
        g.replay()
        torch.cuda.synchronize()
        start.record()
        g.replay()
        end.record()
    else:
        start.record()
        for _ in range(iters):
            fn()
        end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters * 1e3


def bench_gemm(a):
    from . import gemm

    dev = "cuda"
    M, N, K = a.m, a.n, a.k
    # rotate over enough weight copies that the working set exceeds L2 (126 MB)
    nrep = max(1, min(8, int(256e6 // (N * K * 2)) + 1))
    Ws = [torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05 for _ in range(nrep)]
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    i = [0]

    def ours():
        gemm(x, Ws[i[0] % nrep])
        i[0] += 1

    def lib():
        torch.matmul(x, Ws[i[0] % nrep].t())
        i[0] += 1

    out = {"kernel": "gemm_bf16", "M": M, "N": N, "K": K, "weight_copies": nrep}
    us = _time(ours, a.iters, a.warmup)
    out.update(us=round(us, 2), tflops=round(2.0 * M * N * K / us / 1e6, 1),
               gbs=round((N * K + M * K + M * N) * 2 / us / 1e3, 1))
    if a.library:
        us2 = _time(lib, a.iters, a.warmup)
        out.update(library_us=round(us2, 2), library_tflops=round(2.0 * M * N * K / us2 / 1e6, 1))
    return out


def bench_lmhead(a):
    from . import lmhead_logprob_entropy

    dev = "cuda"
    T, H, V = a.t, a.hidden, a.vocab
    h = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    w = torch.randn(V, H, device=dev, dtype=torch.bfloat16) * 0.02
    labels = torch.randint(0, V, (T,), device=dev)
    us = _time(lambda: lmhead_logprob_entropy(h, w, labels, 1.0), a.iters, a.warmup, graph=False)
    hg, wg = h.clone().requires_grad_(True), w.clone().requires_grad_(True)
    g_lp = torch.rand(T, device=dev)

    def fwd_bwd():
        hg.grad = wg.grad = None
        lp, ent = lmhead_logprob_entropy(hg, wg, labels, 1.0)
        lp.backward(g_lp)

    us_fb = _time(fwd_bwd, max(a.iters // 4, 3), a.warmup, graph=False)
    return {"kernel": "lmhead_logprob_fwd", "T": T, "H": H, "V": V, "us": round(us, 1),
            "tflops": round(2.0 * T * H * V / us / 1e6, 1), "fwd_bwd_us": round(us_fb, 1),
            "fwd_bwd_tflops": round(6.0 * T * H * V / us_fb / 1e6, 1)}


def bench_decode(a):
    from . import paged_decode_attention, decode_workspace

    dev = "cuda"
    B, ctx, Hq, Hk, D, bs = a.batch, a.ctx, a.hq, a.hk, 128, a.block_size
    nb_per = (ctx + bs - 1) // bs
    NB = B * nb_per
    kc = torch.randn(NB, Hk, bs, D, device=dev, dtype=torch.bfloat16)
    vc = torch.randn_like(kc)
    bt = torch.randperm(NB, device=dev).int().reshape(B, nb_per)
    lens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    q = torch.randn(B, Hq, D, device=dev, dtype=torch.bfloat16)
    splits = a.splits or decode_workspace(B, Hq, Hk, D, ctx, dev)[0]
    work = torch.empty(B * Hq * splits * (D + 2), device=dev)
    us = _time(lambda: paged_decode_attention(q, kc, vc, bt, lens, num_splits=splits, work=work, impl=a.impl), a.iters,
               a.warmup)
    byts = 2 * B * ctx * Hk * D * 2
    return {"kernel": f"paged_decode_{a.impl}", "B": B, "ctx": ctx, "Hq": Hq, "Hk": Hk, "block_size": bs, "splits": splits,
            "kv_bytes": byts, "us": round(us, 1), "gbs": round(byts / us / 1e3, 1)}


def bench_attn(a):
    """Varlen causal GQA attention forward (7B head layout), ours and (``--library``) flash_attn."""
    from .attention import attention_varlen

    dev = "cuda"
    B, S, Hq, Hk, D = a.batch, a.ctx, a.hq, a.hk, 128
    T = B * S
    qkv = torch.randn(T, (Hq + 2 * Hk) * D, device=dev, dtype=torch.bfloat16)
    q = qkv[:, : Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D : (Hq + Hk) * D].view(T, Hk, D)
    v = qkv[:, (Hq + Hk) * D :].view(T, Hk, D)
    cu = torch.arange(0, T + 1, S, dtype=torch.int32, device=dev)
    flops = 4.0 * B * Hq * D * S * S / 2
    out = {"kernel": "flash_fwd", "B": B, "S": S, "Hq": Hq, "Hk": Hk}
    with torch.no_grad():
        us = _time(lambda: attention_varlen(q, k, v, cu, S, causal=True, impl="native"), a.iters, a.warmup, graph=False)
        out.update(us=round(us, 1), tflops=round(flops / us / 1e6, 1))
        if a.library:
            us2 = _time(lambda: attention_varlen(q, k, v, cu, S, causal=True, impl="library"), a.iters, a.warmup, graph=False)
            out.update(library_us=round(us2, 1), library_tflops=round(flops / us2 / 1e6, 1))
    # backward (dQ, dK, dV; 2.5x the forward FLOPs), ours and the library's
    from . import attention as att

    do = torch.randn(T, Hq, D, device=dev, dtype=torch.bfloat16)
    qg, kg, vg = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    for name in (["native", "library"] if a.library else ["native"]):
        att._BWD_IMPL = name

        def fb():
            o = attention_varlen(qg, kg, vg, cu, S, causal=True, impl="native")
            o.backward(do)
            qg.grad = kg.grad = vg.grad = None

        us3 = _time(fb, a.iters, a.warmup, graph=False)
        key = "fwd_bwd" if name == "native" else "fwd_bwd_library_bwd"
        out[key + "_us"] = round(us3, 1)
        out[key + "_tflops"] = round(3.5 * flops / us3 / 1e6, 1)
    att._BWD_IMPL = "native"
    if a.library:
        # a newer yardstick than flash_attn 2: cuDNN's fused attention through torch SDPA (same shapes, dense batch)
        try:
            from torch.nn.attention import SDPBackend, sdpa_kernel

            qd = q.view(B, S, Hq, D).transpose(1, 2).contiguous().requires_grad_(True)
            kd = k.view(B, S, Hk, D).transpose(1, 2).contiguous().requires_grad_(True)
            vd = v.view(B, S, Hk, D).transpose(1, 2).contiguous().requires_grad_(True)
            dod = do.view(B, S, Hq, D).transpose(1, 2).contiguous()
            sdpa = torch.nn.functional.scaled_dot_product_attention
            with sdpa_kernel(SDPBackend.CUDNN_ATTENTION):
                with torch.no_grad():
                    us4 = _time(lambda: sdpa(qd, kd, vd, is_causal=True, enable_gqa=True), a.iters, a.warmup, graph=False)

                def fb2():
                    o = sdpa(qd, kd, vd, is_causal=True, enable_gqa=True)
                    o.backward(dod)
                    qd.grad = kd.grad = vd.grad = None

                us5 = _time(fb2, a.iters, a.warmup, graph=False)
            out.update(cudnn_sdpa_us=round(us4, 1), cudnn_sdpa_tflops=round(flops / us4 / 1e6, 1),
                       cudnn_sdpa_fwd_bwd_us=round(us5, 1), cudnn_sdpa_fwd_bwd_tflops=round(3.5 * flops / us5 / 1e6, 1))
        except Exception as e:  # backend not available for this shape / build
            out["cudnn_sdpa_error"] = f"{type(e).__name__}: {str(e)[:160]}"
    return out


def bench_decode_step(a):
    """One CUDA-graph decode step of the rollout engine on a model with the 7B layer shapes."""
    from ..models import preset
    from ..models.transformer import CausalLM
    from ..rollout import NativeRolloutEngine, SamplingParams

    dev = torch.device("cuda")
    cfg = preset(a.model, num_hidden_layers=a.layers)
    m = CausalLM(cfg, dtype=torch.bfloat16, device=dev)
    m.init_weights(0)
    eng = NativeRolloutEngine(m, max_num_seqs=a.batch, max_model_len=a.ctx + 64, max_num_batched_tokens=8192,
                              gpu_memory_utilization=0.3)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(100, cfg.vocab_size - 100, (a.ctx - 8,), generator=g).tolist() for _ in range(a.batch)]
    eng.generate(prompts, SamplingParams(temperature=1.0, max_tokens=4, ignore_eos=True))
    st, graph, run = eng._get_graph(a.batch)
    # the sequences above have finished and their rows are padding again: give every row a context of `ctx` tokens
    # (pages spread over the whole cache) and leave it not alive, so that replays do not advance or write the cache
    per = (a.ctx + eng.block_size - 1) // eng.block_size
    nblk = eng.k_cache[0].shape[0]
    st["bt"][:, :per] = (torch.randperm(a.batch * per, device=dev) % nblk).view(a.batch, per).int()
    st["lens"].fill_(a.ctx)
    st["pos"].fill_(a.ctx - 1)
    st["alive"].zero_()
    st["slots"].fill_(-1)
    us = _time(graph.replay, a.iters, a.warmup, graph=False)
    return {"kernel": "decode_step_graph", "model": a.model, "layers": a.layers, "B": a.batch, "ctx": a.ctx,
            "us": round(us, 1), "tokens_per_s": round(a.batch / us * 1e6, 0)}


def bench_fp8_gemm(a):
    """Block-scaled fp8 GEMM (1 x 128 activation scales, 128 x 128 weight scales) next to the bf16 GEMM."""
    from . import fp8, gemm

    M, N, K = a.m, a.n, a.k
    nrep = max(1, min(8, int(256e6 // (N * K)) + 1))
    ws = [fp8.quantize_weight(torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05) for _ in range(nrep)]
    wb = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    xq, sx = fp8.quantize_activation(x)
    i = [0]

    def ours():
        wq, sw = ws[i[0] % nrep]
        fp8.fp8_gemm(xq, sx, wq, sw)
        i[0] += 1

    us = _time(ours, a.iters, a.warmup)
    us_q = _time(lambda: fp8.quantize_activation(x), a.iters, a.warmup)
    us_b = _time(lambda: gemm(x, wb), a.iters, a.warmup)
    return {"kernel": "fp8_gemm_blockscale", "M": M, "N": N, "K": K, "us": round(us, 2), "tflops": round(2.0 * M * N * K / us / 1e6, 1),
            "gbs": round((N * K + M * K + 2 * M * N) / us / 1e3, 1), "act_quant_us": round(us_q, 2), "bf16_gemm_us": round(us_b, 2)}


def bench_grouped_gemm(a):
    """Grouped (MoE) GEMM: ``--batch`` experts, ``--m`` routed rows in total (uniform routing), N x K per expert."""
    from . import moe

    E, T, N, K = a.batch, a.m, a.n, a.k
    top_i = torch.randint(0, E, (T, 1), device="cuda")
    dest, blk_expert, expert_off, P = moe.moe_layout(top_i, E)
    xs = torch.randn(P, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(E, N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    with torch.no_grad():
        us = _time(lambda: moe.grouped_linear(xs, w, blk_expert, expert_off), a.iters, a.warmup)
    return {"kernel": "grouped_gemm_bf16", "experts": E, "rows": T, "padded_rows": P, "N": N, "K": K, "us": round(us, 2),
            "tflops_useful": round(2.0 * T * N * K / us / 1e6, 1), "weight_gbs": round(E * N * K * 2 / us / 1e3, 1)}


def bench_small(a):
    """Every small (bandwidth-bound) kernel once or twice on inputs larger than L2: RMSNorm forward / backward, RoPE,
    SwiGLU forward / backward, embedding forward / backward, AdamW, sum of squares, fused PPO loss, GAE, GRPO advantage,
    sampler, KV-cache write, decode advance, fp8 quantisation. Prints CUDA-event times and effective bandwidths; meant
    to be run under a profiler for per-kernel summaries as well."""
    from . import (adamw_step, decode_advance, embedding, gae, grpo_advantage, kv_cache_write, ppo_loss_fused, rmsnorm,
                   rope_qkv, rope_tables, sample, sumsq_into, swiglu)
    from . import fp8

    dev = "cuda"
    T, H, I = a.t, a.hidden, 18944
    bf = torch.bfloat16
    out = {"kernel": "small_kernels", "T": T, "H": H}

    def timed(name, fn, nbytes):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3
        out[name] = {"us": round(us, 1), "gbs": round(nbytes / us / 1e3, 1)}

    x = torch.randn(T, H, device=dev, dtype=bf, requires_grad=True)
    res = torch.randn(T, H, device=dev, dtype=bf)
    w = torch.ones(H, device=dev, dtype=bf, requires_grad=True)
    timed("rmsnorm_fwd", lambda: rmsnorm(x.detach(), w.detach(), 1e-6, res), 4 * T * H * 2)
    y, hsum = rmsnorm(x, w, 1e-6, res)
    gy = torch.randn_like(y)
    timed("rmsnorm_bwd", lambda: torch.autograd.grad(y, x, gy, retain_graph=True), 3 * T * H * 2)
    Hq, Hk, D = 28, 4, 128
    qkv = torch.randn(T, (Hq + 2 * Hk) * D, device=dev, dtype=bf)
    cos, sin = rope_tables(D, 32768, 1e6, dev)
    pos = torch.arange(T, device=dev) % 4096
    timed("rope", lambda: rope_qkv(qkv, pos, cos, sin, Hq, Hk, D), 2 * T * (Hq + Hk) * D * 2)
    gu = torch.randn(T // 2, 2 * I, device=dev, dtype=bf, requires_grad=True)
    timed("swiglu_fwd", lambda: swiglu(gu.detach()), 3 * (T // 2) * I * 2)
    so = swiglu(gu)
    gso = torch.randn_like(so)
    timed("swiglu_bwd", lambda: torch.autograd.grad(so, gu, gso, retain_graph=True), 5 * (T // 2) * I * 2)
    V = 152064
    emb = torch.randn(V, H, device=dev, dtype=bf, requires_grad=True)
    ids = torch.randint(0, V, (T,), device=dev)
    timed("embedding_fwd", lambda: embedding(ids, emb.detach()), 2 * T * H * 2)
    eo = embedding(ids, emb)
    geo = torch.randn_like(eo)
    timed("embedding_bwd", lambda: torch.autograd.grad(eo, emb, geo, retain_graph=True), T * H * 2 + T * H * 4)
    n = 64 << 20
    p32, g32, m32, v32 = (torch.randn(n, device=dev) for _ in range(4))
    v32.abs_()
    p16 = torch.empty(n, device=dev, dtype=bf)
    timed("adamw", lambda: adamw_step(p32, g32, m32, v32, p16, lr=1e-6, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                                      step=3), n * (4 * 4 + 3 * 4 + 2))
    acc = torch.zeros(1, device=dev)
    timed("sumsq", lambda: sumsq_into(g32, acc), n * 4)
    B, R = 4096, 8192
    lp = -torch.rand(B, R, device=dev)
    lp.requires_grad_(True)
    old, adv, ref = lp.detach() + 0.01, torch.randn(B, R, device=dev), lp.detach() - 0.01
    mask = torch.ones(B, R, device=dev)
    timed("ppo_loss", lambda: ppo_loss_fused(lp, old, adv, mask, ref_logp=ref, kl_coef=0.001), 6 * B * R * 4)
    timed("gae", lambda: gae(adv, old, mask, 1.0, 0.95), 5 * B * R * 4)
    gids = (torch.arange(B, device=dev) // 8).int()
    timed("grpo_adv", lambda: grpo_advantage(adv[:, 0].contiguous(), gids, mask, B // 8), 2 * B * R * 4)
    logits = torch.randn(256, V, device=dev)
    step = torch.zeros(1, dtype=torch.long, device=dev)
    timed("sample", lambda: sample(logits, temperature=torch.ones(256, device=dev), seed=1, step=step), 256 * V * 4)
    NB, bs = 16384, 16
    kc = torch.zeros(NB, Hk, bs, D, device=dev, dtype=bf)
    vc = torch.zeros_like(kc)
    kn, vn = torch.randn(T, Hk, D, device=dev, dtype=bf), torch.randn(T, Hk, D, device=dev, dtype=bf)
    slots = torch.randperm(NB * bs, device=dev)[:T]
    timed("kv_cache_write", lambda: kv_cache_write(kn, vn, slots, kc, vc), 4 * T * Hk * D * 2)
    Bd, mb = 256, 96
    z64 = lambda: torch.zeros(Bd, dtype=torch.long, device=dev)  # noqa: E731
    z32 = lambda v=0: torch.full((Bd,), v, dtype=torch.int32, device=dev)  # noqa: E731
    bt = torch.arange(Bd * mb, device=dev, dtype=torch.int32).view(Bd, mb)
    ring_t, ring_l = torch.zeros(8, Bd, dtype=torch.long, device=dev), torch.zeros(8, Bd, device=dev)
    bpos = torch.zeros(1, dtype=torch.int32, device=dev)
    st = (z64(), torch.zeros(Bd, device=dev), z64(), z64(), z64(), z32(5), bt, 16, z32(1000), z32(1), z32(0), 2, ring_t, ring_l,
          bpos, step)
    timed("decode_advance", lambda: (bpos.zero_(), decode_advance(*st)), Bd * 64)
    wq = torch.randn(18944, 3584, device=dev, dtype=bf)
    timed("fp8_quant_weight", lambda: fp8.quantize_weight(wq), wq.numel() * 3)
    xa = torch.randn(T, H, device=dev, dtype=bf)
    timed("fp8_quant_act", lambda: fp8.quantize_activation(xa), xa.numel() * 3)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "lmhead", "decode", "decode_step", "attn", "fp8_gemm", "grouped_gemm", "small"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--t", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=3584)
    ap.add_argument("--vocab", type=int, default=152064)
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--ctx", type=int, default=900)
    ap.add_argument("--hq", type=int, default=28)
    ap.add_argument("--hk", type=int, default=4)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--impl", default="tc")
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--library", action="store_true")
    a = ap.parse_args(argv)
    fn = {"gemm": bench_gemm, "lmhead": bench_lmhead, "decode": bench_decode, "decode_step": bench_decode_step, "attn": bench_attn,
          "fp8_gemm": bench_fp8_gemm, "grouped_gemm": bench_grouped_gemm, "small": bench_small}[a.what]
    print(json.dumps(fn(a)))


if __name__ == "__main__":
    main()
