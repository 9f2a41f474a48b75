"""Apertus family (two-matrix MLP with the learnable xIELU activation, QK-norm, its own norm names): logits against
``transformers`` on a tiny random model, HF name round trip, greedy rollout and one training step."""

import pytest
import torch


def test_apertus_matches_hf_and_round_trips():
    pytest.importorskip("transformers")
    from transformers import ApertusConfig, ApertusForCausalLM

    from verl_b200.models import CausalLM, PackedBatch
    from verl_b200.models.config import ModelConfig
    from verl_b200.models.hf_io import hf_to_native_state_dict, native_to_hf_state_dict

    hf_cfg = ApertusConfig(vocab_size=512, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
                           num_key_value_heads=2, max_position_embeddings=512, rope_theta=10000.0, rope_scaling=None,
                           tie_word_embeddings=False, rms_norm_eps=1e-5)
    torch.manual_seed(0)
    hf = ApertusForCausalLM(hf_cfg).float().eval()
    with torch.no_grad():  # distinct activation parameters per layer
        for i, layer in enumerate(hf.model.layers):
            layer.mlp.act_fn.alpha_p.add_(0.3 * (i + 1))
            layer.mlp.act_fn.alpha_n.sub_(0.2 * (i + 1))
    d = hf_cfg.to_dict()
    cfg = ModelConfig.from_hf_dict(d)
    assert cfg.model_type == "apertus" and cfg.qk_norm and not cfg.mlp_gated and not cfg.attention_bias
    native = hf_to_native_state_dict(cfg, dict(hf.state_dict()))
    model = CausalLM(cfg, dtype=torch.float32)
    missing, unexpected = model.load_state_dict(native, strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    assert cfg.num_parameters() == sum(p.numel() for p in model.parameters())
    ids = torch.randint(3, 500, (23,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = hf(input_ids=ids[None]).logits[0]
        out = model(PackedBatch(ids, torch.arange(23), torch.tensor([0, 23], dtype=torch.int32), 23))
    torch.testing.assert_close(out, ref, atol=2e-4, rtol=2e-4)
    back = native_to_hf_state_dict(cfg, native)
    ref_sd = dict(hf.state_dict())
    assert set(back) == set(ref_sd), set(back) ^ set(ref_sd)
    for k in ref_sd:
        torch.testing.assert_close(back[k].reshape(ref_sd[k].shape), ref_sd[k])


def test_apertus_rollout_and_training_step():
    from verl_b200.models import CausalLM, PackedBatch, preset
    from verl_b200.rollout import NativeRolloutEngine, SamplingParams
    from verl_b200.workers.engine.native import NativeEngine

    class C(dict):
        __getattr__ = dict.get

    cfg = preset("tiny-apertus")
    eng = NativeEngine(cfg, C(), C(lr=1e-3, clip_grad=1.0), device="cpu", seed=2).initialize()
    roll = NativeRolloutEngine(eng.model, max_num_seqs=4, max_model_len=64, max_num_batched_tokens=64, num_blocks=32)
    prompt = list(range(10, 22))
    out = roll.generate([prompt], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))[0]
    seq = torch.tensor(prompt + out.token_ids)
    with torch.no_grad():
        logits = eng.model(PackedBatch(seq, torch.arange(seq.numel()), torch.tensor([0, seq.numel()], dtype=torch.int32), seq.numel()))
    assert logits[len(prompt) - 1 : -1].argmax(-1).tolist() == out.token_ids  # paged decode = full forward
    batch = PackedBatch(seq, torch.arange(seq.numel()), torch.tensor([0, seq.numel()], dtype=torch.int32), seq.numel())
    rows = torch.arange(seq.numel() - 1)
    before = eng.model.layers[0].mlp.act_alpha_p.detach().clone()
    with eng.train_mode():
        eng.optimizer_zero_grad()
        lp, _ = eng.forward_logprob(batch, rows, seq[1:], 1.0)
        (-lp.mean()).backward()
        gn = float(eng.optimizer_step())
    assert gn > 0 and not torch.equal(eng.model.layers[0].mlp.act_alpha_p.detach(), before)  # the activation trains too
