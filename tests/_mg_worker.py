"""Child process of tests/test_multigpu.py (one rank per GPU, launched through torch.distributed.run)."""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def check_comm(comm, rank, world, dev):
    from verl_b200.ops import _lib

    for it in range(3):
        n = 4096 * 3 + 8 * it
        src = comm.alloc(n, torch.bfloat16)
        src.copy_((torch.arange(n, device=dev) % 251 + rank * 7 + it).to(torch.bfloat16))
        out = torch.empty(n * world, dtype=torch.bfloat16, device=dev)
        exp = torch.cat([(torch.arange(n, device=dev) % 251 + r * 7 + it).to(torch.bfloat16) for r in range(world)])
        for ce in (False, True):  # SM-load kernel and copy-engine variant
            out.zero_()
            comm.all_gather(out, src, copy_engine=ce)
            assert torch.equal(out, exp), f"all_gather mismatch (iteration {it}, copy_engine={ce})"

        shard = 1024 * 5 + 4 * it
        full = comm.alloc(shard * world, torch.float32)
        g = torch.Generator(device="cpu").manual_seed(100 * it + rank)
        full.copy_(torch.randn(shard * world, generator=g).to(dev))
        dst = torch.full((shard,), 0.5, device=dev)
        want = torch.zeros(shard)
        for r in range(world):
            gr = torch.Generator(device="cpu").manual_seed(100 * it + r)
            want += torch.randn(shard * world, generator=gr)[rank * shard : (rank + 1) * shard]
        for nvls in (False, True):
            comm.use_nvls = nvls
            d = dst.clone()
            comm.reduce_scatter_add(d, full, scale=0.25)
            torch.testing.assert_close(d.cpu(), 0.5 + 0.25 * want, atol=1e-5, rtol=1e-5)
        comm.barrier()
    comm.check()
    assert _lib.read_status(dev)[0] == 0


def check_ulysses_a2a(comm, rank, world, dev):
    """The peer-memory all-to-all of the Ulysses exchanges equals the torch.distributed one, in both directions, for
    several rounds (alternating staging buffers), and a decoder layer under sequence parallelism uses it."""
    from verl_b200.utils import ulysses

    Tl, H, D = 96, 4 * world, 128
    for it in range(4):
        g = torch.Generator().manual_seed(10 * it + rank)
        x = torch.randn(Tl, H, D, generator=g).to(dev, torch.bfloat16)
        want = ulysses._all_to_all(x, 1, 0, dist.group.WORLD)           # NCCL: [W Tl, H / W, D]
        got = comm.all_to_all_heads(x, gather_seq=True)
        assert torch.equal(got, want), f"gather-seq exchange differs (round {it})"
        back_want = ulysses._all_to_all(want, 0, 1, dist.group.WORLD)   # [Tl, H, D]
        back = comm.all_to_all_heads(got, gather_seq=False)
        assert torch.equal(back, back_want) and torch.equal(back, x), f"gather-heads exchange differs (round {it})"
    ulysses.register_peer_comm(dist.group.WORLD, comm)
    x = torch.randn(Tl, H, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
    y = ulysses.gather_seq_scatter_heads(x, 0, 1, group=dist.group.WORLD)
    z = ulysses.gather_heads_scatter_seq(y * 2.0, 1, 0, group=dist.group.WORLD)
    z.sum().backward()
    assert torch.equal(z.detach(), (x * 2.0).detach()) and torch.equal(x.grad, torch.full_like(x, 2.0))
    ulysses._PEER_COMMS.clear()
    comm.check()


def check_tp_allreduce(comm, rank, world, dev):
    """Fused all-reduce + residual + RMSNorm over peer memory: bit-identical on all ranks, equal to the fp32 reference,
    also when replayed from a CUDA graph (device-side epoch)."""
    if world not in (2, 4, 8):
        return
    rows, H = 200, 3584
    bufs = [comm.alloc(rows * H, torch.bfloat16, zero=False) for _ in range(2)]
    comm.barrier()
    w = (torch.rand(H, generator=torch.Generator().manual_seed(1)) + 0.5).to(dev, torch.bfloat16)
    res = torch.randn(rows, H, generator=torch.Generator().manual_seed(2)).to(dev, torch.bfloat16)
    parts = [torch.randn(rows, H, generator=torch.Generator().manual_seed(100 + r)).to(torch.bfloat16) for r in range(world)]
    ref_h = (sum(p.float() for p in parts) + res.float().cpu()).to(torch.bfloat16)
    ref_y = (ref_h.float() * torch.rsqrt(ref_h.float().pow(2).mean(-1, keepdim=True) + 1e-6) * w.float().cpu()).to(torch.bfloat16)

    def one(i):
        b = bufs[i & 1][: rows * H].view(rows, H)
        b.copy_(parts[rank].to(dev))
        return comm.tp_allreduce_rmsnorm(b, res, w, 1e-6)

    for i in range(4):
        y, h = one(i)
        torch.testing.assert_close(h.float().cpu(), ref_h.float(), atol=6e-2, rtol=2e-2)
        torch.testing.assert_close(y.float().cpu(), ref_y.float(), atol=6e-2, rtol=2e-2)
        both = [torch.empty_like(h) for _ in range(world)]
        dist.all_gather(both, h)
        assert all(torch.equal(b_, both[0]) for b_ in both), "the ranks' sums differ"
    # replay from a CUDA graph: the kernel advances its own epoch
    stage = [parts[rank].to(dev)]
    g = torch.cuda.CUDAGraph()
    s_ = torch.cuda.Stream()
    s_.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s_):
        outs = []
        for i in range(2):
            b = bufs[i & 1][: rows * H].view(rows, H)
            b.copy_(stage[0])
            outs.append(comm.tp_allreduce_rmsnorm(b, res, w, 1e-6))
    torch.cuda.current_stream().wait_stream(s_)
    torch.cuda.synchronize()
    with torch.cuda.graph(g):
        outs = []
        for i in range(2):
            b = bufs[i & 1][: rows * H].view(rows, H)
            b.copy_(stage[0])
            outs.append(comm.tp_allreduce_rmsnorm(b, res, w, 1e-6))
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    for y, h in outs:
        torch.testing.assert_close(h.float().cpu(), ref_h.float(), atol=6e-2, rtol=2e-2)
    comm.check()


def _packed(ids, lens, dev):
    from verl_b200.models.transformer import PackedBatch

    cu = torch.zeros(len(lens) + 1, dtype=torch.int32, device=dev)
    cu[1:] = torch.cumsum(torch.tensor(lens, device=dev), 0)
    pos = torch.cat([torch.arange(n, device=dev) for n in lens])
    return PackedBatch(ids, pos, cu, max(lens))


def check_reshard(comm, rank, world, dev):
    """ZeRO shards -> full rollout weights (TP = 1) through the one-launch segment copy."""
    from verl_b200.models import preset
    from verl_b200.models.transformer import CausalLM
    from verl_b200.parallel.reshard import RolloutWeights
    from verl_b200.workers.engine.native import NativeEngine

    cfg = preset("tiny-qwen2")
    ref_model = CausalLM(cfg, dtype=torch.bfloat16, device=dev)
    ref_model.init_weights(7)
    ref_state = {k: v.detach().clone() for k, v in ref_model.named_parameters()}
    eng = NativeEngine(cfg, None, None, device=str(dev), group=dist.group.WORLD, seed=7, trainable=False,
                       comm=comm).initialize()
    roll = CausalLM(cfg, dtype=torch.bfloat16, device=dev)
    roll.init_weights(8)
    rw = RolloutWeights(cfg, eng.zero, roll, tp_rank=0, tp_size=1)
    rw.sync()
    torch.cuda.synchronize()
    comm.check()
    n = 0
    for k, v in roll.named_parameters():
        assert torch.equal(v, ref_state[k]), f"reshard mismatch in {k}"
        n += 1
    assert n > 0


def check_zero_step(rank, world, dev, comm):
    """One optimizer step of the native engine: peer-memory collectives vs NCCL collectives give the same weights."""
    from verl_b200.models import preset
    from verl_b200.workers.engine.native import NativeEngine

    class C(dict):
        __getattr__ = dict.get

    cfg = preset("tiny-qwen2")
    optim = C(lr=1e-3, weight_decay=0.01, betas=(0.9, 0.95), clip_grad=1.0, lr_warmup_steps=0, total_training_steps=10)
    outs = []
    # third variant: every layer keeps its activations (no recomputation), over the peer-memory collectives
    for use_comm, keep in ((True, "0"), (False, "0"), (True, str(cfg.num_hidden_layers))):
        eng = NativeEngine(cfg, C(keep_activation_layers=keep), optim, device=str(dev), group=dist.group.WORLD, seed=3,
                           comm=comm if use_comm else None).initialize()
        g = torch.Generator().manual_seed(50 + rank)
        lens = [37, 64, 21]
        ids = torch.randint(0, cfg.vocab_size, (sum(lens),), generator=g).to(dev)
        batch = _packed(ids, lens, dev)
        labels = torch.roll(ids, -1)
        rows = torch.arange(ids.numel(), device=dev)
        with eng.train_mode():
            eng.optimizer_zero_grad()
            lp, ent = eng.forward_logprob(batch, rows, labels, 1.0)
            (-lp.mean()).backward()
            gn = eng.optimizer_step()
        outs.append((float(gn), eng.zero.master.clone().float(), float(lp.mean())))
    (gn_a, w_a, l_a), (gn_b, w_b, l_b), (gn_c, w_c, l_c) = outs
    assert abs(l_a - l_c) < 1e-5 and abs(gn_a - gn_c) <= 1e-4 * max(1.0, abs(gn_a)), (l_a, l_c, gn_a, gn_c)
    torch.testing.assert_close(w_a, w_c, atol=1e-3, rtol=1e-3)
    assert abs(l_a - l_b) < 1e-3, (l_a, l_b)
    assert abs(gn_a - gn_b) <= 2e-3 * max(1.0, abs(gn_b)), (gn_a, gn_b)
    # one AdamW step moves every weight by about lr = 1e-3: the two collective paths must agree to a small fraction of
    # that on nearly all elements (a gradient next to zero may flip the sign of its normalised update)
    diff = (w_a - w_b).abs()
    assert float((diff > 1e-4).float().mean()) < 1e-3 and float(diff.max()) <= 2.5e-3, (float(diff.max()),
                                                                                          float((diff > 1e-4).float().mean()))


def check_ag_gemm(comm, rank, world, dev):
    """Fused all-gather + GEMM against a GEMM on the explicitly gathered weight."""
    from verl_b200 import ops

    torch.manual_seed(21)  # same data on every rank
    M, N, K, w_off = 1000, 1536 + 64, 640, 4096
    total = w_off + N * K + 777
    shard_n = (total + world - 1) // world
    shard_n = (shard_n + 255) // 256 * 256
    flat = torch.zeros(shard_n * world, dtype=torch.bfloat16, device=dev)
    flat[:total] = (torch.randn(total, device=dev) * 0.05).bfloat16()
    shard = comm.alloc(shard_n, torch.bfloat16)
    shard.copy_(flat[rank * shard_n : (rank + 1) * shard_n])
    x = torch.randn(M, K, device=dev).bfloat16()
    bias = torch.randn(N, device=dev).bfloat16()
    W = flat[w_off : w_off + N * K].view(N, K)
    for it in range(2):
        out, w_full = comm.ag_gemm(x, shard, w_off, N, K, bias=bias)
        torch.cuda.synchronize()
        comm.check()
        assert torch.equal(w_full, W), "gathered weight differs"
        ref = ops.gemm(x, W, bias=bias)
        assert torch.equal(out, ref), "fused result differs from the plain GEMM on the same weight"
        comm.barrier()


def check_gemm_rs(comm, rank, world, dev):
    """Fused GEMM -> reduce-scatter (row-parallel linear) against the fp32 sum of all ranks' products, for a
    prefill-like and a decode-like (split-K) shape; and a sequence-parallel MLP block built from the TP layers."""
    from verl_b200.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear

    for M, N, K in ((1024, 1536, 640), (128, 3584, 2048)):
        g = torch.Generator(device="cpu").manual_seed(100 + M)
        xs = [(torch.randn(M, K, generator=g) * 0.5).bfloat16() for _ in range(world)]  # every rank's K-slice
        ws = [(torch.randn(N, K, generator=g) * 0.05).bfloat16() for _ in range(world)]
        res = torch.randn(M, N, generator=g).bfloat16()
        want = sum(x.float() @ w.float().t() for x, w in zip(xs, ws)) + res.float()
        rows = M // world
        x, w = xs[rank].to(dev), ws[rank].to(dev)
        mine = res[rank * rows:(rank + 1) * rows].to(dev).contiguous()
        for it in range(3):  # repeated calls: the two receive buffers alternate
            out = comm.gemm_rs(x, w, residual=mine)
            torch.cuda.synchronize()
            comm.check()
            ref = want[rank * rows:(rank + 1) * rows].to(dev)
            err = (out.float() - ref).abs().max().item()
            assert err < 0.02 * ref.abs().max().item() + 0.05, (M, N, K, it, err)
    # column-parallel -> SwiGLU-free elementwise -> row-parallel, against the unsharded computation
    g = torch.Generator(device="cpu").manual_seed(7)
    M, H, I = 64 * world, 512, 1024 * world
    x_full = (torch.randn(M, H, generator=g) * 0.5).bfloat16()
    w1 = (torch.randn(I, H, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(H, I, generator=g) * 0.05).bfloat16()
    want = (torch.relu(x_full.float() @ w1.float().t()).bfloat16().float() @ w2.float().t())
    ip, rows = I // world, M // world
    col = ColumnParallelLinear(comm, w1[rank * ip:(rank + 1) * ip].to(dev).contiguous())
    row = RowParallelLinear(comm, w2[:, rank * ip:(rank + 1) * ip].to(dev).contiguous())
    y = row(torch.relu(col(x_full[rank * rows:(rank + 1) * rows].to(dev).contiguous())))
    torch.cuda.synchronize()
    comm.check()
    ref = want[rank * rows:(rank + 1) * rows].to(dev)
    assert (y.float() - ref).abs().max().item() < 0.03 * ref.abs().max().item() + 0.05
    comm.barrier()


def check_moe_ep(comm, rank, world, dev):
    """Expert-parallel MoE (dispatch -> grouped GEMMs on the owners -> combine) against every expert evaluated in
    fp32 on this rank's own tokens. Two rounds with different routings reuse the buffers."""
    from verl_b200 import ops
    from verl_b200.parallel.expert_parallel import ExpertParallelMoE

    E, H, I, k, T = 4 * world, 512, 256, 2, 300
    g = torch.Generator(device="cpu").manual_seed(11)
    gate_up = (torch.randn(E, 2 * I, H, generator=g) * 0.05).bfloat16()
    down = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16()
    El = E // world
    gu_l, dn_l = gate_up[rank * El:(rank + 1) * El].to(dev).contiguous(), down[rank * El:(rank + 1) * El].to(dev).contiguous()
    ep = ExpertParallelMoE(comm, E, H, k, max_tokens=T)
    for rnd in range(2):
        gr = torch.Generator(device="cpu").manual_seed(100 * rnd + rank)
        n_tok = T - 37 * rank - 11 * rnd  # ranks hold different numbers of tokens
        x = (torch.randn(n_tok, H, generator=gr) * 0.5).bfloat16()
        logits = torch.randn(n_tok, E, generator=gr)
        if rnd == 1:
            logits[:, 0] += 4.0  # skewed routing: most tokens on expert 0 (rank 0)
        top_w, top_i = torch.softmax(logits, -1).topk(k, -1)
        out = ep.forward(x.to(dev), top_i.to(dev), top_w.to(dev), gu_l, dn_l, ops.swiglu)
        torch.cuda.synchronize()
        comm.check()
        ref = torch.zeros(n_tok, H)
        for j in range(k):
            for e in range(E):
                m = top_i[:, j] == e
                if m.any():
                    hgu = (x[m].float() @ gate_up[e].float().t()).bfloat16().float()
                    act = (torch.nn.functional.silu(hgu[:, :I]) * hgu[:, I:]).bfloat16().float()
                    ref[m] += top_w[m, j, None] * (act @ down[e].float().t()).bfloat16().float()
        err = (out.float().cpu() - ref).abs().max().item()
        assert err < 0.02 * ref.abs().max().item() + 0.02, (rnd, err, ref.abs().max().item())
    comm.barrier()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from verl_b200.parallel.peer_comm import PeerComm

    comm = PeerComm(dist.group.WORLD)
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    if what in ("comm", "all"):
        check_comm(comm, rank, world, dev)
    if what in ("reshard", "all"):
        check_reshard(comm, rank, world, dev)
    if what in ("ag_gemm", "all"):
        check_ag_gemm(comm, rank, world, dev)
    if what in ("moe_ep", "all"):
        check_moe_ep(comm, rank, world, dev)
    if what in ("gemm_rs", "all"):
        check_gemm_rs(comm, rank, world, dev)
    if what in ("zero", "all"):
        check_zero_step(rank, world, dev, comm)
    if what in ("ulysses_a2a", "all"):
        check_ulysses_a2a(comm, rank, world, dev)
    if what in ("tp_allreduce", "all"):
        check_tp_allreduce(comm, rank, world, dev)
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print(f"MG_WORKER_OK {what}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
