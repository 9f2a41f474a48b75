"""Burst decode (several decode steps chained on the device, the host reads their tokens in one go) gives exactly what
step-by-step decoding gives: same tokens, log-probs and stop reasons, with sequences that end inside a burst by EOS or
by their length limit, with more requests than slots, and with a KV cache too small for everything at once."""

import pytest
import torch

from verl_b200.models import CausalLM, preset
from verl_b200.rollout import NativeRolloutEngine, SamplingParams


def _run(model, prompts, sps, burst, **kw):
    args = dict(max_num_seqs=8, max_model_len=96, max_num_batched_tokens=64, num_blocks=96, seed=3, decode_burst=burst)
    args.update(kw)
    eng = NativeRolloutEngine(model, **args)
    out = eng.generate(prompts, sps)
    return [(o.token_ids, o.log_probs, o.stop_reason) for o in out], eng.stats


@pytest.mark.parametrize("temperature", [0.0, 1.0])
def test_burst_matches_single_steps(temperature):
    cfg = preset("tiny-qwen2", vocab_size=64)  # small vocabulary: the EOS id is sampled often
    model = CausalLM(cfg, dtype=torch.float32).init_weights(1)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, 64, (n,), generator=g).tolist() for n in (5, 9, 14, 3, 7, 11, 6, 8, 10, 4, 12)]
    lens = [30, 7, 19, 25, 1, 13, 40, 9, 16, 22, 5]  # limits that fall inside bursts
    sps = [SamplingParams(temperature=temperature, max_tokens=n) for n in lens]
    sps[2] = SamplingParams(temperature=temperature, max_tokens=19, ignore_eos=True)
    ref, st1 = _run(model, prompts, sps, 1)
    for burst, kw in ((8, {}), (5, {"num_blocks": 24}), (16, {"max_num_seqs": 3})):
        got, st = _run(model, prompts, sps, burst, **kw)
        if not kw:
            assert st["steps"] < st1["steps"]  # far fewer host round trips
        if temperature == 0.0:  # greedy streams do not depend on who shares the batch (sampled ones draw per batch row)
            assert [(g[0], g[2]) for g in got] == [(r[0], r[2]) for r in ref]
            for g_, r_ in zip(got, ref):
                torch.testing.assert_close(torch.tensor(g_[1]), torch.tensor(r_[1]), atol=1e-4, rtol=1e-4)
        for (toks, lps, why), sp in zip(got, sps):
            assert 1 <= len(toks) <= sp.max_tokens and len(lps) == len(toks)
            if why == "completed":
                assert toks[-1] == cfg.eos_token_id and not sp.ignore_eos
            else:
                assert why == "length" and len(toks) == sp.max_tokens
            assert sp.ignore_eos or cfg.eos_token_id not in toks[:-1]
    assert any(why == "length" for _, _, why in ref)
    if temperature > 0:  # the sampled streams do hit EOS (1 of 64 ids), also in the middle of bursts
        assert any(why == "completed" for _, _, why in ref) and any(why == "completed" for _, _, why in got)


def test_greedy_eos_inside_a_burst():
    cfg = preset("tiny-qwen2", vocab_size=64)
    model = CausalLM(cfg, dtype=torch.float32).init_weights(1)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(3, 64, (n,), generator=g).tolist() for n in (5, 9, 14, 3, 7, 11)]
    sp = SamplingParams(temperature=0.0, max_tokens=24)
    free, _ = _run(model, prompts, sp, 1, eos_token_id=1)
    eos = free[2][0][5]  # a token that the third greedy stream emits in the middle of the first burst
    ref, _ = _run(model, prompts, sp, 1, eos_token_id=eos)
    got, _ = _run(model, prompts, sp, 8, eos_token_id=eos)
    assert [(a[0], a[2]) for a in got] == [(b[0], b[2]) for b in ref]
    assert ref[2][2] == "completed" and len(ref[2][0]) <= 6
