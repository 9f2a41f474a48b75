"""Multi-GPU micro-benchmarks of the peer-memory collectives and the fused compute + collective kernels.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m verl_b200.parallel.microbench {collectives,ag_gemm,gemm_rs,moe_ep}

Device time from CUDA events after warm-up, maximum over ranks. Every fused kernel is printed next to its unfused
form (our GEMM, then the collective) and the NCCL collective, with the roofline figure: the slower of FLOPs over the
measured GEMM rate of the same shape on one GPU and bytes that must cross NVLink over 770 GB/s per direction.
"""

from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def _timeit(fn, dev, iters=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def bench_collectives(comm, rank, world, dev):
    n = 233_000_000 // world // 256 * 256  # one 7B decoder layer
    src = comm.alloc(n, torch.bfloat16)
    out = torch.empty(n * world, dtype=torch.bfloat16, device=dev)
    for ce in (False, True):
        t = _timeit(lambda: comm.all_gather(out, src, copy_engine=ce), dev)
        if rank == 0:
            print(f"peer all_gather copy_engine={ce} {n * 2 * world / 1e6:.0f} MB: {t:.3f} ms, "
                  f"{n * 2 * (world - 1) / t / 1e6:.1f} GB/s in per GPU")
    t = _timeit(lambda: dist.all_gather_into_tensor(out, src), dev)
    if rank == 0:
        print(f"nccl all_gather: {t:.3f} ms, {n * 2 * (world - 1) / t / 1e6:.1f} GB/s")
    full = comm.alloc(n * world, torch.float32)
    dst = torch.zeros(n, device=dev)
    t = _timeit(lambda: comm.reduce_scatter_add(dst, full), dev)
    if rank == 0:
        print(f"peer reduce_scatter_add {n * 4 * world / 1e6:.0f} MB: {t:.3f} ms, {n * 4 * (world - 1) / t / 1e6:.1f} GB/s in per GPU")
    tmp = torch.empty(n, device=dev)
    t = _timeit(lambda: dist.reduce_scatter_tensor(tmp, full), dev)
    if rank == 0:
        print(f"nccl reduce_scatter: {t:.3f} ms, {n * 4 * (world - 1) / t / 1e6:.1f} GB/s")


def bench_ag_gemm(comm, rank, world, dev):
    from .. import ops

    for M, N, K in ((16384, 37888, 3584), (16384, 4608, 3584), (4096, 37888, 3584)):
        shard_n = (N * K + world - 1) // world // 256 * 256 + 256
        shard = comm.alloc(shard_n, torch.bfloat16)
        shard.normal_(0, 0.02)
        x = torch.randn(M, K, device=dev).bfloat16()
        wfull = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
        gath = torch.empty(shard_n * world, dtype=torch.bfloat16, device=dev)
        fused = _timeit(lambda: comm.ag_gemm(x, shard, 0, N, K, w_full=wfull), dev, iters=5)

        def separate():
            comm.all_gather(gath, shard, copy_engine=True)
            ops.gemm(x, gath[: N * K].view(N, K))

        sep = _timeit(separate, dev, iters=5)
        alone = _timeit(lambda: ops.gemm(x, wfull), dev, iters=5)
        link = N * K * 2 * (world - 1) / world / (NVLINK_GBS * 1e6)
        if rank == 0:
            print(f"ag_gemm M={M} N={N} K={K}: fused {fused:.3f} ms, gather-then-gemm {sep:.3f} ms, gemm alone {alone:.3f} ms, "
                  f"link {link:.3f} ms -> roofline {max(alone, link):.3f} ms, fused reaches {max(alone, link) / fused:.2f}")


def bench_gemm_rs(comm, rank, world, dev):
    """Row-parallel projections of the 7B architecture with the contraction split over the ranks: o_proj and
    down_proj for a prefill chunk of 8192 tokens and a decode step of 128 * world tokens."""
    from .. import ops

    for M, N, Kfull in ((8192, 3584, 18944), (8192, 3584, 3584), (128 * world, 3584, 18944), (128 * world, 3584, 3584)):
        K = Kfull // world // 64 * 64
        x = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
        rows = M // world
        fused = _timeit(lambda: comm.gemm_rs(x, w), dev)
        full = comm.alloc(M * N, torch.float32, zero=False)
        dst = torch.zeros(rows * N, device=dev)

        def separate():  # our GEMM into symmetric memory, then our pull reduce-scatter
            ops.gemm(x, w, out=full.view(M, N))
            dst.zero_()
            comm.reduce_scatter_add(dst, full)

        sep = _timeit(separate, dev)
        y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        o = torch.empty(rows, N, dtype=torch.bfloat16, device=dev)

        def nccl():
            ops.gemm(x, w, out=y)
            dist.reduce_scatter_tensor(o, y)

        t_nccl = _timeit(nccl, dev)
        alone = _timeit(lambda: ops.gemm(x, w, out=y), dev)
        link = M * N * 2 * (world - 1) / world / (NVLINK_GBS * 1e6)
        if rank == 0:
            print(f"gemm_rs M={M} N={N} K={K}/rank: fused {fused * 1e3:.1f} us, gemm + peer reduce-scatter {sep * 1e3:.1f} us, "
                  f"gemm + nccl reduce-scatter {t_nccl * 1e3:.1f} us, gemm alone {alone * 1e3:.1f} us, link {link * 1e3:.1f} us "
                  f"-> roofline {max(alone, link) * 1e3:.1f} us, fused reaches {max(alone, link) / fused:.2f}")
    comm.check()


def bench_moe_ep(comm, rank, world, dev):
    """Expert-parallel MoE layer of the Qwen3-30B-A3B architecture (hidden 2048, 128 experts, top-8, expert
    intermediate 768): whole layer, and its communication (dispatch + combine) next to NCCL all-to-alls of the same
    payload (uniform random routing)."""
    from .. import ops
    from .expert_parallel import ExpertParallelMoE

    E, H, I, k = 128, 2048, 768, 8
    El = E // world
    gate_up = (torch.randn(El, 2 * I, H, device=dev) * 0.02).bfloat16()
    down = (torch.randn(El, H, I, device=dev) * 0.02).bfloat16()
    for T in (4096, 128):
        ep = ExpertParallelMoE(comm, E, H, k, max_tokens=T, capacity_rows=2 * T * k + El * 127)
        x = (torch.randn(T, H, device=dev) * 0.5).bfloat16()
        top_w, top_i = torch.softmax(torch.randn(T, E, device=dev), -1).topk(k, -1)
        layer = _timeit(lambda: ep.forward(x, top_i, top_w, gate_up, down, ops.swiglu), dev)
        comm.check()

        def comm_only():  # layout + dispatch + handshake + combine (the experts' output buffer is read as it is)
            ti, tw = top_i.to(torch.int32), top_w.float()
            base, _, _ = ep.layout(ti)
            where = torch.empty(T * k, dtype=torch.int32, device=dev)
            ep.lib.vb_moe_dispatch(x.data_ptr(), ti.data_ptr(), T, k, H, El, base.data_ptr(), ep.cursor.data_ptr(),
                                   ep._recv_ptrs, world, where.data_ptr(), ep.cap, comm._status(), _stream())
            comm.barrier()
            out = torch.empty_like(x)
            ep.lib.vb_moe_combine(ep._y_ptrs, comm.pad_alloc.ptrs, ti.data_ptr(), tw.data_ptr(), where.data_ptr(), T, k, H, El,
                                  out.data_ptr(), rank, world, comm.CH_COPY, comm._epoch(comm.CH_COPY),
                                  comm._gate(comm.CH_COPY), comm._status(), _stream())

        t_comm = _timeit(comm_only, dev)
        rows = T * k
        send = torch.empty(rows, H, dtype=torch.bfloat16, device=dev)
        recv = torch.empty_like(send)

        def nccl():
            dist.all_to_all_single(recv, send)
            dist.all_to_all_single(send, recv)

        t_nccl = _timeit(nccl, dev)
        remote = rows * H * 2 * (world - 1) / world  # bytes leaving (dispatch) and entering (combine) this GPU
        link = 2 * remote / (NVLINK_GBS * 1e6)
        if rank == 0:
            print(f"moe_ep T={T}/rank: layer {layer * 1e3:.1f} us, dispatch+combine {t_comm * 1e3:.1f} us "
                  f"({2 * remote / t_comm / 1e6:.0f} GB/s over NVLink, link-time {link * 1e3:.1f} us = {link / t_comm:.2f}), "
                  f"two NCCL all-to-alls of the same payload {t_nccl * 1e3:.1f} us")


def _stream():
    return torch.cuda.current_stream().cuda_stream


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from .peer_comm import PeerComm

    comm = PeerComm(dist.group.WORLD)
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm_rs"
    {"collectives": bench_collectives, "ag_gemm": bench_ag_gemm, "gemm_rs": bench_gemm_rs, "moe_ep": bench_moe_ep}[what](comm, rank, world, dev)
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
