"""Native model vs HF transformers on CPU (fp32): same weights -> same logits / log-probs."""
import pytest
import torch

from verl_b200.models import PackedBatch, build_model, preset
from verl_b200.models.hf_io import hf_to_native_state_dict, native_to_hf_state_dict


def _hf_model(cfg, kind):
    import transformers

    d = {k: v for k, v in cfg.to_hf_dict().items() if k not in ("architectures", "torch_dtype", "extra")}
    if kind == "qwen2":
        hc = transformers.Qwen2Config(**d)
        return transformers.Qwen2ForCausalLM(hc).float().eval()
    if kind == "llama":
        hc = transformers.LlamaConfig(**d)
        return transformers.LlamaForCausalLM(hc).float().eval()
    if kind == "qwen3":
        hc = transformers.Qwen3Config(**d)
        return transformers.Qwen3ForCausalLM(hc).float().eval()
    raise ValueError(kind)


@pytest.mark.parametrize("kind", ["qwen2", "llama", "qwen3"])
def test_logits_match_hf(kind):
    torch.manual_seed(0)
    cfg = preset("tiny-qwen2", model_type=kind, tie_word_embeddings=(kind == "qwen2"))
    if kind == "qwen3":
        cfg = preset("tiny-qwen2", model_type="qwen3", head_dim=64, tie_word_embeddings=False)
    hf = _hf_model(cfg, kind)
    with torch.no_grad():
        for p in hf.parameters():
            p.normal_(0, 0.05)
    m = build_model(cfg, dtype=torch.float32, init=False)
    missing, unexpected = m.load_state_dict(hf_to_native_state_dict(cfg, hf.state_dict()), strict=False)
    assert not unexpected and all("lm_head" in k for k in missing), (missing, unexpected)
    ids = torch.randint(0, cfg.vocab_size, (3, 19))
    mask = torch.ones(3, 19, dtype=torch.long)
    mask[1, 12:] = 0
    mask[2, 5:] = 0
    batch, idx = PackedBatch.from_padded(ids, mask)
    with torch.no_grad():
        ref = hf(input_ids=ids, attention_mask=mask).logits.reshape(-1, cfg.vocab_size)[idx]
        got = m(batch)
    torch.testing.assert_close(got, ref, atol=2e-4, rtol=2e-4)
    # round trip of the name mapping
    back = native_to_hf_state_dict(cfg, m.state_dict())
    for k, v in hf.state_dict().items():
        if k == "lm_head.weight" and cfg.tie_word_embeddings:
            continue
        torch.testing.assert_close(back[k], v)


def test_fused_logprob_matches_logits_path():
    torch.manual_seed(0)
    cfg = preset("tiny-qwen2")
    m = build_model(cfg, dtype=torch.float32)
    ids = torch.randint(0, cfg.vocab_size, (2, 11))
    batch, _ = PackedBatch.from_padded(ids, torch.ones_like(ids))
    labels = torch.roll(batch.input_ids, -1)
    lp, ent = m(batch, labels, temperature=0.7)
    logits = m(batch) / 0.7
    ref = torch.log_softmax(logits, -1).gather(1, labels[:, None])[:, 0]
    torch.testing.assert_close(lp, ref, atol=1e-5, rtol=1e-5)
    p = torch.softmax(logits, -1)
    torch.testing.assert_close(ent, -(p * torch.log(p)).sum(-1), atol=1e-4, rtol=1e-4)
