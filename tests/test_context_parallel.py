"""Context parallelism: zig-zag layout, chunk-pair attention against full causal attention (values and gradients,
ranks emulated in one process), and a 2-rank engine step against the unsharded engine (gloo)."""

import os
import subprocess
import sys

import pytest
import torch


def _full_and_cp(lens, cp, Hq=4, Hk=2, D=16, seed=0, device="cpu", dtype=torch.float32):
    from verl_b200 import ops
    from verl_b200.parallel.context_parallel import cp_attention_local, cp_local_index

    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    q, k, v = (torch.randn(T, h, D, generator=g).to(device=device, dtype=dtype).requires_grad_(True) for h in (Hq, Hk, Hk))
    w = torch.randn(T, Hq, D, generator=g).to(device=device, dtype=dtype)
    ref = ops.attention_varlen(q, k, v, cu.to(device), max(lens), causal=True)
    gref = torch.autograd.grad((ref.float() * w.float()).sum(), (q, k, v))

    idxs = [cp_local_index(cu, r, cp) for r in range(cp)]
    cu_chunk = idxs[0][1].to(device)
    Tc = int(cu_chunk[-1])

    def take(x, idx):  # padding rows read token 0 of the stream (any finite values do)
        return torch.where((idx >= 0).view(-1, 1, 1), x[idx.clamp(min=0)], torch.zeros_like(x[:1]) + 0.1)

    # keys / values in global chunk order, as the all-gather + reorder delivers them
    k_chunks, v_chunks = [None] * (2 * cp), [None] * (2 * cp)
    for r in range(cp):
        idx = idxs[r][0].to(device)
        kl, vl = take(k, idx), take(v, idx)
        k_chunks[r], k_chunks[2 * cp - 1 - r] = kl[:Tc], kl[Tc:]
        v_chunks[r], v_chunks[2 * cp - 1 - r] = vl[:Tc], vl[Tc:]
    k_all, v_all = torch.cat(k_chunks), torch.cat(v_chunks)
    out = torch.zeros_like(ref)
    for r in range(cp):
        idx = idxs[r][0].to(device)
        o = cp_attention_local(take(q, idx), k_all, v_all, cu_chunk, int((cu_chunk[1:] - cu_chunk[:-1]).max()), r, cp)
        valid = idx >= 0
        out = out.index_put((idx[valid],), o[valid].to(out.dtype))
    gcp = torch.autograd.grad((out.float() * w.float()).sum(), (q, k, v))
    return ref, out, gref, gcp


@pytest.mark.parametrize("lens,cp", [([16, 8], 2), ([13, 5, 1, 22], 2), ([9, 30], 4), ([7], 3)])
def test_chunk_pair_attention_matches_full_causal_attention(lens, cp):
    from verl_b200.parallel.context_parallel import cp_local_index

    ref, out, gref, gcp = _full_and_cp(lens, cp)
    assert torch.allclose(out, ref, atol=1e-5), float((out - ref).abs().max())
    for a, b in zip(gcp, gref):
        assert torch.allclose(a, b, atol=1e-5), float((a - b).abs().max())
    # layout: every token is held by exactly one rank; chunks are equal per sequence; ranks hold the same count
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    held = torch.cat([cp_local_index(cu, r, cp)[0] for r in range(cp)])
    assert sorted(held[held >= 0].tolist()) == list(range(sum(lens)))
    assert len({cp_local_index(cu, r, cp)[0].numel() for r in range(cp)}) == 1


@pytest.mark.timeout(600)
def test_engine_step_with_context_parallelism_matches_unsharded():
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29700 + os.getpid() % 90), os.path.join(here, "_cp_train_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=560)
    assert r.returncode == 0 and "CP_TRAIN_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-3000:])


@pytest.mark.gpu
@pytest.mark.parametrize("lens,cp", [([256, 130], 2), ([700, 64, 1], 4)])
def test_chunk_pair_attention_on_the_kernels(lens, cp):
    """The tcgen05 path: forward merged through the parts' log-sum-exp, backward = the flash backward of every chunk
    pair with the merged output and the global log-sum-exp. Against the same kernels on the whole sequences."""
    ref, out, gref, gcp = _full_and_cp(lens, cp, Hq=8, Hk=2, D=128, device="cuda", dtype=torch.bfloat16)
    scale = float(ref.float().abs().max())
    assert float((out.float() - ref.float()).abs().max()) <= 0.03 * scale
    for a, b in zip(gcp, gref):
        s = float(b.float().abs().max())
        assert float((a.float() - b.float()).abs().max()) <= 0.04 * s + 1e-3


@pytest.mark.timeout(600)
def test_update_actor_with_context_parallelism_under_spmd_launch():
    """The worker path (batch pooling inside the group, mini-batch normalisation, dispatch registration): update_actor
    with context_parallel_size=2 equals the data-parallel update over the same samples."""
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29800 + os.getpid() % 90), os.path.join(here, "_sp_spmd_worker.py"), "cp"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=560)
    assert r.returncode == 0 and "SP_SPMD_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-3000:])
