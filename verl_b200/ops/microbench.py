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


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "lmhead", "decode", "decode_step", "attn", "fp8_gemm", "grouped_gemm"])
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
          "fp8_gemm": bench_fp8_gemm, "grouped_gemm": bench_grouped_gemm}[a.what]
    print(json.dumps(fn(a)))


if __name__ == "__main__":
    main()
