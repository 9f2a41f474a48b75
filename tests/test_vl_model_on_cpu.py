"""Qwen2-VL family: the native vision tower + multimodal RoPE decoder against HF ``transformers`` on a tiny random
model (logits of a sequence with an image), the position-id builder, and HF name round trips."""

import pytest
import torch

from verl_b200.models import CausalLM, PackedBatch
from verl_b200.models.config import ModelConfig
from verl_b200.models.hf_io import hf_to_native_state_dict, native_to_hf_state_dict
from verl_b200.models.vision import get_rope_index


def _hf_tiny():
    from transformers import Qwen2VLConfig, Qwen2VLForConditionalGeneration

    cfg = Qwen2VLConfig(
        text_config=dict(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]},
                         max_position_embeddings=512, tie_word_embeddings=False, rope_theta=10000.0),
        vision_config=dict(depth=2, embed_dim=32, hidden_size=64, num_heads=2, mlp_ratio=2, in_channels=3, patch_size=4,
                           spatial_merge_size=2, temporal_patch_size=2),
        image_token_id=500, video_token_id=501, vision_start_token_id=502, tie_word_embeddings=False)
    torch.manual_seed(0)
    m = Qwen2VLForConditionalGeneration(cfg).float().eval()
    return cfg, m


def test_vl_logits_match_hf_and_names_round_trip():
    pytest.importorskip("transformers")
    hf_cfg, hf = _hf_tiny()
    cfg = ModelConfig.from_hf_dict(hf_cfg.to_dict())
    assert cfg.is_vl and cfg.mrope_section == [2, 3, 3] and cfg.image_token_id == 500 and cfg.hidden_size == 64
    native = hf_to_native_state_dict(cfg, dict(hf.state_dict()))
    model = CausalLM(cfg, dtype=torch.float32)
    missing, unexpected = model.load_state_dict(native, strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    # one image of 1 x 4 x 4 patches -> 4 placeholder tokens after the 2 x 2 merge
    grid = torch.tensor([[1, 4, 4]])
    g = torch.Generator().manual_seed(1)
    pixels = torch.randn(16, 3 * 2 * 4 * 4, generator=g)
    ids = torch.tensor([5, 9, 502, 500, 500, 500, 500, 7, 11, 13, 17])
    pos3, delta = get_rope_index(ids, grid, image_token_id=500, spatial_merge_size=2)
    with torch.no_grad():
        mm = (ids == 500).int()[None]  # 0 = text, 1 = image placeholder
        am = torch.ones(1, ids.numel(), dtype=torch.long)
        ref = hf(input_ids=ids[None], pixel_values=pixels, image_grid_thw=grid, attention_mask=am, mm_token_type_ids=mm)
        hf_pos, hf_delta = hf.model.get_rope_index(ids[None], mm, image_grid_thw=grid, attention_mask=am)
        batch = PackedBatch(ids, pos3, torch.tensor([0, ids.numel()], dtype=torch.int32), ids.numel(), pixel_values=pixels,
                            image_grid_thw=grid)
        logits = model(batch)
    assert torch.equal(pos3, hf_pos[:, 0]) and delta == int(hf_delta.flatten()[0])
    torch.testing.assert_close(logits, ref.logits[0], atol=2e-4, rtol=2e-4)
    # text-only sequences of a VL model keep working (all three axes advance together)
    p1, d1 = get_rope_index(torch.tensor([5, 6, 7]), None, 500)
    assert torch.equal(p1, torch.arange(3).expand(3, 3)) and d1 == 0
    back = native_to_hf_state_dict(cfg, native)
    ref_sd = dict(hf.state_dict())
    assert set(back) == set(ref_sd)
    for k in ref_sd:
        assert torch.equal(back[k], ref_sd[k]), k
