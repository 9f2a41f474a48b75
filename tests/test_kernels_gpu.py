"""Numerics of every hand-written CUDA kernel against a plain PyTorch fp32 reference of the same op.

Tolerances: outputs stored in bf16 are compared with rtol ~ 2 bf16 ulps of the reference magnitude;
fp32 outputs (log-probs, entropy, optimizer state) with the tolerances the reference uses for its
fused kernels (tests/utils/test_linear_cross_entropy.py: logprob atol 1e-3 / rtol 2e-4, entropy atol 5e-3).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _bf16_close(got, ref, scale=None, ulps=4.0):
    got, ref = got.float(), ref.float().to(got.device)
    scale = ref.abs().max().item() if scale is None else scale
    err = (got - ref).abs().max().item()
    assert err <= ulps * 2 ** -8 * scale + 1e-6, f"max err {err} vs scale {scale}"


@pytest.fixture(autouse=True)
def _status_clean():
    from verl_b200.ops import _lib

    _lib.load()
    yield
    code, blk, detail = _lib.read_status()
    assert code == 0, f"kernel status word reports error {code} (block {blk}, detail {detail})"


@pytest.mark.parametrize("mode", ["tn", "nn", "wg", "an"])
@pytest.mark.parametrize("shape", [(128, 256, 64), (200, 264, 136), (1024, 3584, 3584), (777, 128, 1000),
                                   (8, 1024, 512), (384, 72, 256)])
def test_gemm_layouts(mode, shape):
    from verl_b200.ops import gemm

    torch.manual_seed(0)
    M, N, K = shape
    a_mn, b_mn = {"tn": (False, False), "nn": (False, True), "wg": (True, True), "an": (True, False)}[mode]
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operand needs a row stride that is a multiple of 8")
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    ref = A.float() @ B.float().t()
    out = gemm(A.t().contiguous() if a_mn else A, B.t().contiguous() if b_mn else B, a_mn=a_mn, b_mn=b_mn)
    _bf16_close(out, ref)


def test_gemm_fp32_accumulate_and_bias():
    from verl_b200.ops import gemm

    torch.manual_seed(1)
    M, N, K = 256, 520, 384
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    C = torch.full((M, N), 3.0, device="cuda")
    gemm(A, B, out=C, accumulate=True)
    torch.testing.assert_close(C, A.float() @ B.float().t() + 3.0, atol=1e-3, rtol=1e-5)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    _bf16_close(gemm(A, B, bias=bias), A.float() @ B.float().t() + bias.float())


@pytest.mark.parametrize("M,N,K,mode", [(128, 3584, 18944, "tn"), (64, 4608, 3584, "tn"), (7, 520, 2048, "tn"),
                                        (128, 1024, 4096, "nn"), (200, 640, 8192, "tn"), (128, 3584, 3584, "tn"),
                                        (256, 2304, 3584, "tn"), (128, 4608, 3584, "tn"), (100, 1796, 1800, "tn")])
def test_gemm_split_k(M, N, K, mode):
    """Skinny problems split K: over the CTAs of a cluster with the reduction through distributed shared memory
    (uneven row shares when the slice count does not divide 128, ragged N and K), or, with fp32 accumulation into C,
    over fp32 slices in a workspace. Same numbers as the fp32 reference, bit-identical between calls, bias handled by
    the reducing CTA."""
    from verl_b200.ops import gemm, _lib

    torch.manual_seed(3)
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    ref = A.float() @ B.float().t()
    Bm = B.t().contiguous() if mode == "nn" else B
    o1 = gemm(A, Bm, b_mn=(mode == "nn"), bias=bias)
    o2 = gemm(A, Bm, b_mn=(mode == "nn"), bias=bias)
    assert _lib.read_status("cuda")[0] == 0
    _bf16_close(o1, ref + bias.float())
    assert torch.equal(o1, o2)
    C = torch.full((M, N), 2.0, device="cuda")
    gemm(A, Bm, b_mn=(mode == "nn"), out=C, accumulate=True)
    torch.testing.assert_close(C, ref + 2.0, atol=2e-2, rtol=1e-4)


@pytest.mark.parametrize("mode", ["tn", "nn", "wg", "an"])
def test_gemm_cta_pair_path(mode):
    """Large problems run on CTA pairs (256 x 256 tiles, one MMA for two SMs). Odd 128-row block count, ragged N and
    K, every operand layout, bias and fp32 accumulation."""
    from verl_b200.ops import gemm, _lib

    torch.manual_seed(4)
    M, N, K = 4224, 2632, 584
    a_mn, b_mn = {"tn": (False, False), "nn": (False, True), "wg": (True, True), "an": (True, False)}[mode]
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.1
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    ref = A.float() @ B.float().t()
    Am = A.t().contiguous() if a_mn else A
    Bm = B.t().contiguous() if b_mn else B
    out = gemm(Am, Bm, a_mn=a_mn, b_mn=b_mn, bias=bias)
    assert _lib.read_status("cuda")[0] == 0
    _bf16_close(out, ref + bias.float())
    assert torch.equal(out, gemm(Am, Bm, a_mn=a_mn, b_mn=b_mn, bias=bias))
    C = torch.full((M, N), -1.0, device="cuda")
    gemm(Am, Bm, a_mn=a_mn, b_mn=b_mn, out=C, accumulate=True)
    torch.testing.assert_close(C, ref - 1.0, atol=2e-2, rtol=1e-4)


def test_gemm_deterministic():
    from verl_b200.ops import gemm

    A = torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(768, 1024, device="cuda", dtype=torch.bfloat16)
    assert torch.equal(gemm(A, B), gemm(A, B))


def test_linear_autograd_matches_torch():
    from verl_b200 import ops

    torch.manual_seed(2)
    x = torch.randn(300, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(264, 512, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    b = torch.randn(264, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn(300, 264, device="cuda", dtype=torch.bfloat16)
    ops.linear(x, w, b).backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    torch.nn.functional.linear(xr, wr, br).backward(dy.float())
    _bf16_close(x.grad, xr.grad)
    _bf16_close(w.grad, wr.grad)
    _bf16_close(b.grad, br.grad)
    # fused accumulation into an fp32 main_grad
    w2 = w.detach().clone().requires_grad_(True)
    w2.main_grad = torch.ones(w2.shape, device="cuda")
    ops.linear(x.detach(), w2, None).backward(dy)
    assert w2.grad is None
    torch.testing.assert_close(w2.main_grad, wr.grad + 1.0, atol=2e-3, rtol=1e-4)


@pytest.mark.parametrize("T,H,V,temp", [(300, 256, 2048, 1.0), (1937, 3584, 152064, 0.7), (129, 1024, 32000, 1.5)])
def test_fused_lmhead_forward_backward(T, H, V, temp):
    from verl_b200 import ops

    torch.manual_seed(3)
    hid = torch.randn(T, H, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(V, H, device="cuda") * 0.02).bfloat16().requires_grad_(True)
    labels = torch.randint(0, V, (T,), device="cuda")
    lp, ent = ops.lmhead_logprob_entropy(hid, w, labels, temp)
    hr, wr = hid.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    logits = (hr @ wr.t()) / temp
    lse = torch.logsumexp(logits, -1)
    lp_ref = logits.gather(1, labels[:, None])[:, 0] - lse
    ent_ref = lse - (torch.softmax(logits, -1) * logits).sum(-1)
    torch.testing.assert_close(lp, lp_ref, atol=1e-3, rtol=2e-4)
    torch.testing.assert_close(ent, ent_ref, atol=5e-3, rtol=1e-3)
    g_lp = torch.randn(T, device="cuda")
    g_ent = torch.randn(T, device="cuda") * 0.1
    (lp * g_lp + ent * g_ent).sum().backward()
    (lp_ref * g_lp + ent_ref * g_ent).sum().backward()
    _bf16_close(hid.grad, hr.grad, ulps=8)
    _bf16_close(w.grad, wr.grad, ulps=8)


def test_rmsnorm_forward_backward():
    from verl_b200 import ops

    torch.manual_seed(4)
    rows, H = 1000, 3584
    x = torch.randn(rows, H, device="cuda").bfloat16().requires_grad_(True)
    res = torch.randn(rows, H, device="cuda").bfloat16().requires_grad_(True)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16().requires_grad_(True)
    y, h = ops.rmsnorm(x, w, 1e-6, res)
    dy, dh = torch.randn_like(y), torch.randn_like(h)
    torch.autograd.backward([y, h], [dy, dh])
    xr, rr, wr = (t.detach().float().requires_grad_(True) for t in (x, res, w))
    hr = (xr + rr) + ((xr + rr).bfloat16().float() - (xr + rr)).detach()  # bf16-rounded value, identity gradient
    yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    torch.autograd.backward([yr, hr], [dy.float(), dh.float()])
    _bf16_close(y, yr)
    _bf16_close(h, hr)
    _bf16_close(x.grad, xr.grad)
    _bf16_close(res.grad, rr.grad)
    _bf16_close(w.grad, wr.grad, ulps=8)


def test_swiglu_and_rope():
    from verl_b200 import ops

    torch.manual_seed(5)
    gu = torch.randn(512, 2 * 1184, device="cuda").bfloat16().requires_grad_(True)
    do = torch.randn(512, 1184, device="cuda").bfloat16()
    out = ops.swiglu(gu)
    out.backward(do)
    gr = gu.detach().float().requires_grad_(True)
    ref = torch.nn.functional.silu(gr[:, :1184]) * gr[:, 1184:]
    ref.backward(do.float())
    _bf16_close(out, ref)
    _bf16_close(gu.grad, gr.grad)

    T, Hq, Hk, D = 333, 28, 4, 128
    qkv = torch.randn(T, (Hq + 2 * Hk) * D, device="cuda").bfloat16()
    pos = torch.randint(0, 4096, (T,), device="cuda")
    cos_t, sin_t = ops.rope_tables(D, 4096, 1e6, "cuda")
    ref = ops.rope_qkv(qkv.cpu().float(), pos.cpu(), cos_t.cpu(), sin_t.cpu(), Hq, Hk, D)
    src = qkv.clone().requires_grad_(True)
    got = ops.rope_qkv(src * 1.0, pos, cos_t, sin_t, Hq, Hk, D)
    _bf16_close(got, ref)
    # backward is the transpose rotation: <rope(x), g> == <x, rope^T(g)>
    g = torch.randn_like(got)
    got.backward(g)
    lhs = (got.float() * g.float()).sum()
    rhs = (qkv.float() * src.grad.float()).sum()
    assert abs(lhs.item() - rhs.item()) <= 2e-2 * abs(lhs.item()) + 1.0


def test_embedding_and_adamw_and_norms():
    from verl_b200 import ops

    torch.manual_seed(6)
    W = torch.randn(5000, 512, device="cuda").bfloat16().requires_grad_(True)
    ids = torch.randint(0, 5000, (777,), device="cuda")
    out = ops.embedding(ids, W)
    assert torch.equal(out, W[ids])
    dy = torch.randn_like(out)
    out.backward(dy)
    ref = torch.zeros(5000, 512, device="cuda").index_add_(0, ids, dy.float())
    _bf16_close(W.grad, ref)

    n = 1_000_003
    p32, g = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    pr = torch.nn.Parameter(p32.clone())
    opt = torch.optim.AdamW([pr], lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    for step in (1, 2, 3):
        pr.grad = g.clone()
        opt.step()
        ops.adamw_step(p32, g, m, v, p16, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, step=step)
    torch.testing.assert_close(p32, pr.data, atol=2e-6, rtol=1e-5)
    _bf16_close(p16, pr.data)
    ss = torch.zeros(1, device="cuda")
    ops.sumsq_into(g, ss)
    torch.testing.assert_close(ss[0], g.pow(2).sum(), rtol=1e-4, atol=0)
    scale, skip, norm = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda", dtype=torch.int32), torch.zeros(1, device="cuda")
    ops.clip_coef(ss, 1.0, 0.5, scale, skip, norm)
    gn = g.norm().item() * 0.5
    assert abs(norm.item() - gn) < 1e-2 and skip.item() == 0 and abs(scale.item() - 0.5 / (gn + 1e-6)) < 1e-6


def test_ppo_loss_fused_matches_torch():
    from verl_b200 import ops
    from verl_b200.trainer.ppo import core_algos

    torch.manual_seed(7)
    B, T = 16, 200
    logp = (torch.randn(B, T, device="cuda") * 0.5 - 2).requires_grad_(True)
    old = logp.detach() + torch.randn(B, T, device="cuda") * 0.3
    ref_lp = logp.detach() + torch.randn(B, T, device="cuda") * 0.2
    adv = torch.randn(B, T, device="cuda")
    mask = (torch.rand(B, T, device="cuda") > 0.3).float()
    ent = torch.rand(B, T, device="cuda").requires_grad_(True)
    loss, sums = ops.ppo_loss_fused(logp, old, adv, mask, entropy=ent, ref_logp=ref_lp, clip_low=0.2, clip_high=0.28,
                                    clip_c=3.0, kl_coef=0.01, kl_type="low_var_kl", entropy_coeff=0.001)
    loss.backward()
    lr, er = logp.detach().clone().requires_grad_(True), ent.detach().clone().requires_grad_(True)
    pg, clipfrac, ppo_kl, clipfrac_lower = core_algos.compute_policy_loss(
        old, lr, adv, mask, cliprange=0.2, cliprange_low=0.2, cliprange_high=0.28, clip_ratio_c=3.0,
        loss_agg_mode="token-mean")
    kld = core_algos.kl_penalty(lr, ref_lp, "low_var_kl")
    kl_loss = core_algos.agg_loss(kld, mask, "token-mean")
    ent_loss = core_algos.agg_loss(er, mask, "token-mean")
    ref_loss = pg - 0.001 * ent_loss + 0.01 * kl_loss
    ref_loss.backward()
    torch.testing.assert_close(loss, ref_loss, atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(logp.grad, lr.grad, atol=1e-7, rtol=1e-3)
    torch.testing.assert_close(ent.grad, er.grad, atol=1e-8, rtol=1e-3)
    n = sums[6]
    torch.testing.assert_close(sums[1] / n, clipfrac, atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(sums[2] / n, ppo_kl, atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(sums[3] / n, clipfrac_lower, atol=1e-5, rtol=1e-4)


def test_gae_and_grpo_match_core_algos():
    from verl_b200 import ops
    from verl_b200.trainer.ppo import core_algos

    torch.manual_seed(8)
    B, T = 37, 129
    r, v = torch.randn(B, T, device="cuda"), torch.randn(B, T, device="cuda")
    mk = (torch.rand(B, T, device="cuda") > 0.2).float()
    adv, ret = ops.gae(r, v, mk, 0.99, 0.95)
    adv_ref, ret_ref = core_algos.compute_gae_advantage_return(r.cpu(), v.cpu(), mk.cpu(), 0.99, 0.95, whiten=False)
    torch.testing.assert_close(adv.cpu(), adv_ref, atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(ret.cpu(), ret_ref, atol=1e-4, rtol=1e-4)

    import numpy as np

    scores_tok = torch.zeros(B, T)
    scores = torch.randn(B)
    lens = mk.cpu().sum(-1).long().clamp(min=1)
    gid = torch.randint(0, 9, (B,))
    gid[0] = 20  # singleton group
    for b in range(B):
        scores_tok[b, 0] = scores[b]
    ref, _ = core_algos.compute_grpo_outcome_advantage(scores_tok, mk.cpu(), np.array(gid.tolist()))
    got = ops.grpo_advantage(scores.cuda(), gid.cuda(), mk, 21)
    torch.testing.assert_close(got.cpu(), ref, atol=1e-4, rtol=1e-4)


def test_sampler_distribution_and_modes():
    from verl_b200 import ops

    torch.manual_seed(9)
    V, n = 1000, 4096
    logits = torch.randn(1, V, device="cuda").repeat(n, 1).contiguous()
    step = torch.zeros(1, device="cuda", dtype=torch.long)
    tok, lp = ops.sample(logits, seed=1234, step=step)
    p = torch.softmax(logits[0], -1)
    freq = torch.bincount(tok, minlength=V).float() / n
    assert (freq - p).abs().sum().item() / 2 < 0.25
    torch.testing.assert_close(lp, torch.log(p)[tok], atol=1e-5, rtol=1e-5)
    tok2, _ = ops.sample(logits, seed=1234, step=step)
    assert torch.equal(tok, tok2)  # same seed and step -> same draw
    step += 1
    tok3, _ = ops.sample(logits, seed=1234, step=step)
    assert not torch.equal(tok, tok3)
    tok, _ = ops.sample(logits, temperature=torch.zeros(n, device="cuda"), seed=1, step=step)
    assert bool((tok == logits[0].argmax()).all())
    tok, lp = ops.sample(logits, top_k=torch.full((n,), 5, device="cuda", dtype=torch.int32), seed=7, step=step)
    top5 = logits[0].topk(5)
    assert set(tok.unique().tolist()) <= set(top5.indices.tolist())
    torch.testing.assert_close(lp, torch.log_softmax(top5.values, -1)[(tok[:, None] == top5.indices[None]).float().argmax(-1)],
                               atol=1e-4, rtol=1e-4)
    tok, _ = ops.sample(logits, top_p=torch.full((n,), 0.5, device="cuda"), seed=7, step=step)
    sp, si = p.sort(descending=True)
    kk = int((sp.cumsum(0) < 0.5).sum().item()) + 1
    assert set(tok.unique().tolist()) <= set(si[:kk].tolist())
    # bf16 logits
    tok, _ = ops.sample(logits.bfloat16(), temperature=torch.zeros(n, device="cuda"), seed=1, step=step)
    assert bool((tok == logits[0].bfloat16().float().argmax()).all())


@pytest.mark.parametrize("B,Hq,Hk,D,bs,maxlen", [(5, 28, 4, 128, 16, 700), (3, 4, 2, 64, 16, 300), (2, 32, 4, 128, 32, 3000),
                                                 (4, 40, 8, 128, 16, 150), (3, 32, 2, 128, 128, 1000),
                                                 (2, 8, 8, 128, 8, 260),
                                                 # more (sequence, head, split) items than resident CTAs: the
                                                 # persistent kernel (CTAs walk several items, some of them empty)
                                                 (100, 28, 4, 128, 16, 700), (80, 32, 8, 128, 16, 300)])
def test_paged_decode_attention(B, Hq, Hk, D, bs, maxlen):
    from verl_b200 import ops

    torch.manual_seed(10)
    lens = torch.randint(1, maxlen, (B,), dtype=torch.int32)
    lens[0] = maxlen
    nblk_per = (maxlen + bs - 1) // bs
    NB = B * nblk_per + 3
    kc = torch.zeros(NB, Hk, bs, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    table = torch.randperm(NB)[: B * nblk_per].reshape(B, nblk_per).int().cuda()
    # fill through the cache-write kernel
    for b in range(B):
        L = int(lens[b])
        k_new = torch.randn(L, Hk, D, device="cuda").bfloat16()
        v_new = torch.randn(L, Hk, D, device="cuda").bfloat16()
        pos = torch.arange(L, device="cuda")
        slots = table[b].long()[pos // bs] * bs + pos % bs
        ops.kv_cache_write(k_new, v_new, slots, kc, vc)
    q = torch.randn(B, Hq, D, device="cuda").bfloat16()
    ref = ops.paged_decode_attention(q.cpu().float(), kc.cpu().float(), vc.cpu().float(), table.cpu(), lens)
    from verl_b200.ops import _lib

    impls = ["simt"] if Hq // Hk <= 8 else []
    if _lib.fn("vb_paged_decode_tc_supported")(Hq, Hk, D, bs):
        impls.append("tc")
    assert impls
    for impl in impls:
        for splits in sorted({1, 3, ops.decode_workspace(B, Hq, Hk, D, maxlen, "cuda")[0]}):
            out = ops.paged_decode_attention(q, kc, vc, table, lens.cuda(), num_splits=splits, impl=impl)
            assert _lib.read_status("cuda")[0] == 0
            _bf16_close(out, ref, ulps=4)


def _attn_ref(q, k, v, cu, causal, scale):
    """fp32 reference, one sequence at a time. Returns (out [T,Hq,D], lse [Hq,T])."""
    T, Hq, D = q.shape
    G = Hq // k.shape[1]
    out = torch.empty(T, Hq, D, device=q.device)
    lse = torch.empty(Hq, T, device=q.device)
    b = cu.tolist()
    for s, e in zip(b[:-1], b[1:]):
        qs = q[s:e].float().transpose(0, 1)
        ks = k[s:e].float().repeat_interleave(G, dim=1).transpose(0, 1)
        vs = v[s:e].float().repeat_interleave(G, dim=1).transpose(0, 1)
        sc = qs @ ks.transpose(1, 2) * scale
        if causal:
            n = e - s
            sc = sc.masked_fill(torch.triu(torch.ones(n, n, device=q.device, dtype=torch.bool), 1), float("-inf"))
        lse[:, s:e] = torch.logsumexp(sc, -1)
        out[s:e] = (torch.softmax(sc, -1) @ vs).transpose(0, 1)
    return out, lse


@pytest.mark.parametrize("lens,Hq,Hk,causal", [([300, 77, 512, 129], 28, 4, True), ([1, 128, 640], 8, 8, True),
                                               ([1000, 333], 16, 2, False), ([2048], 4, 4, True)])
def test_flash_attention_fwd(lens, Hq, Hk, causal):
    from verl_b200.ops import _lib
    from verl_b200.ops.attention import flash_fwd

    torch.manual_seed(11)
    D, T = 128, sum(lens)
    # q / k / v as views of one fused buffer (token stride (Hq + 2 Hk) * D), the way the model produces them
    qkv = torch.randn(T, (Hq + 2 * Hk) * D, device="cuda").bfloat16()
    q = qkv[:, : Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D : (Hq + Hk) * D].view(T, Hk, D)
    v = qkv[:, (Hq + Hk) * D :].view(T, Hk, D)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    scale = D ** -0.5
    out, lse = flash_fwd(q, k, v, cu, max(lens), causal, scale)
    assert _lib.read_status("cuda")[0] == 0
    ref, ref_lse = _attn_ref(q, k, v, cu, causal, scale)
    _bf16_close(out, ref, ulps=4)
    torch.testing.assert_close(lse, ref_lse, atol=2e-3, rtol=1e-4)


@pytest.mark.parametrize("lens,Hq,Hk,causal", [([200, 131, 64], 8, 2, True), ([513, 1], 4, 4, True), ([300, 77], 28, 4, True),
                                               ([260], 4, 2, False)])
def test_flash_attention_autograd_matches_reference(lens, Hq, Hk, causal):
    from verl_b200 import ops
    from verl_b200.ops import _lib

    torch.manual_seed(12)
    D = 128
    T = sum(lens)
    q = torch.randn(T, Hq, D, device="cuda").bfloat16().requires_grad_(True)
    k = torch.randn(T, Hk, D, device="cuda").bfloat16().requires_grad_(True)
    v = torch.randn(T, Hk, D, device="cuda").bfloat16().requires_grad_(True)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    do = torch.randn(T, Hq, D, device="cuda").bfloat16()
    ops.attention_varlen(q, k, v, cu, max(lens), causal=causal, impl="native").backward(do)
    assert _lib.read_status("cuda")[0] == 0
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref, _ = _attn_ref(qr, kr, vr, cu, causal, D ** -0.5)
    ref.backward(do.float())
    for got, want in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        err = (got.float() - want).abs().max().item()
        assert err <= 2e-2 * max(1.0, want.abs().max().item()), err


def test_flash_attention_fwd_with_cached_prefix():
    """Queries are the last positions of a longer key stream (chunked prefill on top of cached context)."""
    from verl_b200.ops.attention import flash_fwd

    torch.manual_seed(13)
    Hq, Hk, D = 8, 2, 128
    lq, lk = [100, 1, 260], [100, 300, 700]
    q = torch.randn(sum(lq), Hq, D, device="cuda").bfloat16()
    k = torch.randn(sum(lk), Hk, D, device="cuda").bfloat16()
    v = torch.randn(sum(lk), Hk, D, device="cuda").bfloat16()
    cu_q = torch.tensor([0] + list(torch.tensor(lq).cumsum(0)), dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0] + list(torch.tensor(lk).cumsum(0)), dtype=torch.int32, device="cuda")
    out, _ = flash_fwd(q, k, v, cu_q, max(lq), True, D ** -0.5, cu_seqlens_k=cu_k)
    G = Hq // Hk
    for b in range(len(lq)):
        qs = q[cu_q[b]:cu_q[b + 1]].float().transpose(0, 1)
        ks = k[cu_k[b]:cu_k[b + 1]].float().repeat_interleave(G, 1).transpose(0, 1)
        vs = v[cu_k[b]:cu_k[b + 1]].float().repeat_interleave(G, 1).transpose(0, 1)
        s = qs @ ks.transpose(1, 2) * D ** -0.5
        mask = torch.arange(lk[b], device="cuda")[None, :] <= (torch.arange(lq[b], device="cuda")[:, None] + lk[b] - lq[b])
        ref = (torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ vs).transpose(0, 1)
        _bf16_close(out[cu_q[b]:cu_q[b + 1]], ref, ulps=4)


def test_moe_grouped_gemm_matches_expert_loop():
    """Grouped GEMM path of the MoE MLP (one launch per projection, device-side routing layout) against the
    per-expert fp32 reference: outputs, input gradients, weight gradients (also fused into main_grad)."""
    from verl_b200 import ops
    from verl_b200.ops.moe import moe_mlp

    torch.manual_seed(14)
    T, H, I, E, k = 300, 256, 192, 8, 2
    x = torch.randn(T, H, device="cuda").bfloat16().requires_grad_(True)
    gate_up = (torch.randn(E, 2 * I, H, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    down = (torch.randn(E, H, I, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    logits = torch.randn(T, E, device="cuda")
    logits[:, 5] = -1e9  # an expert without tokens
    top_w, top_i = torch.topk(torch.softmax(logits, -1), k, -1)
    top_w = (top_w / top_w.sum(-1, keepdim=True)).detach()
    dy = torch.randn(T, H, device="cuda").bfloat16()
    y = moe_mlp(x, top_i, top_w, gate_up, down, ops.swiglu)
    y.backward(dy)
    xr, gr, dr = (t.detach().float().requires_grad_(True) for t in (x, gate_up, down))
    ref = torch.zeros(T, H, device="cuda")
    for j in range(k):
        for e in range(E):
            sel = top_i[:, j] == e
            if sel.any():
                gu = xr[sel] @ gr[e].t()
                h = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
                ref[sel] = ref[sel] + (h @ dr[e].t()) * top_w[sel, j : j + 1].float()
    ref.backward(dy.float())

    def close(a, b, tol):
        err = (a.float() - b).abs().max().item()
        assert err <= tol * max(1.0, b.abs().max().item()), (err, b.abs().max().item())

    close(y, ref.detach(), 2e-2)
    close(x.grad, xr.grad, 3e-2)
    close(gate_up.grad, gr.grad, 3e-2)
    close(down.grad, dr.grad, 3e-2)
    assert float(gate_up.grad[5].abs().sum()) == 0.0
    # fused accumulation into fp32 main_grad
    g2 = gate_up.detach().clone().requires_grad_(True)
    g2.main_grad = torch.ones(g2.shape, device="cuda")
    moe_mlp(x.detach(), top_i, top_w, g2, down.detach(), ops.swiglu).backward(dy)
    assert g2.grad is None
    close(g2.main_grad - 1.0, gr.grad, 3e-2)


def test_bounded_device_wait_reports_status_and_context_survives():
    """A cross-rank barrier whose peer never arrives: the kernel gives up after its time limit, records the wait in
    the status word and returns; the host reads the code and the context keeps working."""
    import ctypes
    import time

    from verl_b200.ops import _lib, gemm

    lib = _lib.load()
    lib.vb_peer_barrier.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_uint, ctypes.c_void_p,
                                    ctypes.c_void_p]
    lib.vb_peer_barrier.restype = ctypes.c_int
    _lib.clear_status("cuda")
    mine = torch.zeros(1024, dtype=torch.int32, device="cuda")
    absent = torch.zeros(1024, dtype=torch.int32, device="cuda")  # stands for a peer that never writes its slot
    pads = (ctypes.c_void_p * 2)(mine.data_ptr(), absent.data_ptr())
    t0 = time.perf_counter()
    rc = lib.vb_peer_barrier(pads, 0, 2, 3, 1, _lib.status_word("cuda").data_ptr(), _lib.stream())
    assert rc == 0
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    code, _, detail = _lib.read_status("cuda")
    assert code == 5 and detail == 1, (code, detail)   # ERR_WAIT_FLAG, waiting for rank 1
    assert 1.0 < dt < 10.0
    _lib.clear_status("cuda")
    a = torch.randn(256, 256, device="cuda").bfloat16()
    _bf16_close(gemm(a, a), a.float() @ a.float().t())


@pytest.mark.parametrize("M,N,K,pow2", [(128, 512, 1024, False), (300, 384 + 64, 640, True), (1000, 256, 3584, False)])
def test_fp8_blockscale_quant_and_gemm(M, N, K, pow2):
    from verl_b200.ops import _lib, fp8

    torch.manual_seed(15)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    wq, sw = fp8.quantize_weight(w, pow2)
    xq, sx = fp8.quantize_activation(x, pow2)
    # quantisation agrees with the plain PyTorch statement of the scheme
    wq_ref, sw_ref = fp8.quantize_weight(w.cpu(), pow2)
    xq_ref, sx_ref = fp8.quantize_activation(x.cpu(), pow2)
    torch.testing.assert_close(sw.cpu(), sw_ref, rtol=1e-6, atol=0)
    torch.testing.assert_close(sx.cpu(), sx_ref, rtol=1e-6, atol=0)
    for got, want in ((wq, wq_ref), (xq, xq_ref)):
        a, b = got.cpu().float(), want.float()
        # the kernel multiplies by a fast reciprocal: values next to a rounding boundary may land on the neighbouring
        # e4m3 code (one step = 1/8 relative), nothing may be further off
        assert (a != b).float().mean() < 0.02
        assert ((a - b).abs() <= 0.126 * torch.maximum(a.abs(), b.abs()) + 2 ** -9).all()
    if pow2:
        assert torch.equal(torch.log2(sw), torch.log2(sw).round())
    # GEMM against the dequantised fp32 product, and loosely against the unquantised one
    out = fp8.fp8_gemm(xq, sx, wq, sw, bias)
    assert _lib.read_status("cuda")[0] == 0
    ref = fp8.dequantize(xq, sx, False) @ fp8.dequantize(wq, sw, True).t() + bias.float()
    _bf16_close(out, ref, ulps=4)
    full = x.float() @ w.float().t() + bias.float()
    rel = (out.float() - full).norm() / full.norm()
    assert rel < 0.06, float(rel)
    _bf16_close(fp8.fp8_linear(x, wq, sw, bias, pow2), ref, ulps=4)


@pytest.mark.parametrize("T", [8, 128, 1000])
def test_programmatic_dependent_launch_chain_is_bit_identical(T):
    """A decode-layer-shaped chain (norm -> GEMM -> rope -> cache write -> paged attention -> GEMM -> norm -> GEMM ->
    swiglu -> GEMM) gives the same bits whether each kernel waits for the one before it at launch (the ordinary
    stream order) or only before its first global access (programmatic dependent launch), eagerly and in a graph."""
    from verl_b200 import ops
    from verl_b200.ops import _lib

    torch.manual_seed(3)
    H, Hq, Hk, D, I, bs = 1024, 8, 2, 128, 2048, 16
    dev = "cuda"
    x0 = torch.randn(T, H, device=dev).bfloat16()
    wn = torch.randn(H, device=dev).bfloat16()
    wqkv = (torch.randn((Hq + 2 * Hk) * D, H, device=dev) * 0.03).bfloat16()
    wo = (torch.randn(H, Hq * D, device=dev) * 0.03).bfloat16()
    wgu = (torch.randn(2 * I, H, device=dev) * 0.03).bfloat16()
    wd = (torch.randn(H, I, device=dev) * 0.03).bfloat16()
    ctx = 200
    nblk = (ctx + bs) // bs + 1
    kc = torch.randn(T * nblk, Hk, bs, D, device=dev).bfloat16()
    vc = torch.randn_like(kc)
    table = torch.arange(T * nblk, device=dev, dtype=torch.int32).reshape(T, nblk)
    lens = torch.full((T,), ctx + 1, device=dev, dtype=torch.int32)
    pos = torch.full((T,), ctx, device=dev, dtype=torch.long)
    slots = table[:, ctx // bs].long() * bs + ctx % bs
    cos, sin = ops.rope_tables(D, 4096, 10000.0, dev)

    def chain(x):
        for _ in range(3):
            h, res = ops.rmsnorm(x, wn, 1e-6, None)
            qkv = ops.gemm(h, wqkv)
            qkv = ops.rope_qkv(qkv, pos, cos, sin, Hq, Hk, D)
            q = qkv[:, : Hq * D].view(T, Hq, D)
            k = qkv[:, Hq * D : (Hq + Hk) * D].view(T, Hk, D)
            v = qkv[:, (Hq + Hk) * D :].view(T, Hk, D)
            ops.kv_cache_write(k, v, slots, kc, vc)
            a = ops.paged_decode_attention(q, kc, vc, table, lens)
            o = ops.gemm(a.reshape(T, Hq * D), wo)
            h, res = ops.rmsnorm(o, wn, 1e-6, res)
            x = ops.gemm(ops.swiglu(ops.gemm(h, wgu)), wd)
        return x

    outs = {}
    try:
        for on in (False, True):
            _lib.set_pdl(on)
            outs[on, "eager"] = chain(x0).clone()
            g = torch.cuda.CUDAGraph()
            static_in = x0.clone()
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                chain(static_in)
            torch.cuda.current_stream().wait_stream(s)
            with torch.cuda.graph(g):
                static_out = chain(static_in)
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            outs[on, "graph"] = static_out.clone()
    finally:
        _lib.set_pdl(True)
    ref = outs[False, "eager"]
    assert torch.isfinite(ref.float()).all()
    for key, val in outs.items():
        assert torch.equal(val, ref), f"{key} differs from the ordinary stream order"


def test_kernels_write_inside_their_buffers():
    """Every output and workspace that the ops allocate sits between canary bands while a battery of kernels runs on
    tile-edge shapes; no band may change (the sanitizer-free memory-safety check of this code base)."""
    from verl_b200 import ops
    from verl_b200.utils.debug.guard_bands import guard_allocations

    torch.manual_seed(5)
    dev = "cuda"
    with guard_allocations() as g:
        for M, N, K in [(1, 72, 64), (127, 136, 200), (129, 264, 72), (300, 4608, 512), (8, 3584, 1024)]:
            a = torch.randn(M, K, device=dev).bfloat16()
            w = torch.randn(N, K, device=dev).bfloat16()
            ops.gemm(a, w)
            ops.gemm(a, w, out_dtype=torch.float32)
        for T, H in [(1, 64), (37, 1000), (130, 3584)]:
            x = torch.randn(T, H, device=dev).bfloat16()
            wn = torch.randn(H, device=dev).bfloat16()
            y, r = ops.rmsnorm(x, wn, 1e-6, x)
            ops.swiglu(torch.randn(T, 2 * 256, device=dev).bfloat16())
        Hq, Hk, D, bs = 8, 2, 128, 16
        for T in (1, 33, 200):
            qkv = torch.randn(T, (Hq + 2 * Hk) * D, device=dev).bfloat16()
            cos, sin = ops.rope_tables(D, 2048, 10000.0, dev)
            qkv = ops.rope_qkv(qkv, torch.arange(T, device=dev), cos, sin, Hq, Hk, D)
            q = qkv[:, : Hq * D].view(T, Hq, D)
            k = qkv[:, Hq * D : (Hq + Hk) * D].view(T, Hk, D)
            v = qkv[:, (Hq + Hk) * D :].view(T, Hk, D)
            cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
            ops.attention_varlen(q.contiguous(), k.contiguous(), v.contiguous(), cu, T, causal=True)
        B, ctx = 5, 77
        nblk = (ctx + bs - 1) // bs
        kc = torch.zeros(B * nblk + 2, Hk, bs, D, device=dev, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        table = torch.arange(B * nblk, device=dev, dtype=torch.int32).reshape(B, nblk)
        lens = torch.tensor([ctx, 1, 16, 17, 64], device=dev, dtype=torch.int32)
        knew = torch.randn(B, Hk, D, device=dev).bfloat16()
        slots = table[torch.arange(B, device=dev), ((lens - 1) // bs).long()].long() * bs + ((lens - 1) % bs).long()
        ops.kv_cache_write(knew, knew, slots, kc, vc)
        q1 = torch.randn(B, Hq, D, device=dev).bfloat16()
        for splits in (1, 3):
            ops.paged_decode_attention(q1, kc, vc, table, lens, num_splits=splits)
        logits = torch.randn(7, 1001, device=dev)
        ops.sample(logits, temperature=torch.ones(7, device=dev), seed=3)
        h = torch.randn(100, 256, device=dev).bfloat16()
        wl = (torch.randn(1000, 256, device=dev) * 0.05).bfloat16()
        ops.lmhead_logprob_entropy(h, wl, torch.randint(0, 1000, (100,), device=dev), 1.0)
        n_checked = g.check()
    assert n_checked >= 30
