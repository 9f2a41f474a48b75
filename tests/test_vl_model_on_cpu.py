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


@pytest.mark.parametrize("name", ["tiny-qwen2-vl", "tiny-qwen3-vl"])
def test_vl_batch_through_engine_and_actor(name):
    """A padded batch with one image per sample: the actor's log-probs (multi_modal_inputs + [b, 4, S] position ids through
    the ZeRO engine) equal a direct forward of the same model, and an update step trains the vision tower too."""
    from verl_b200 import DataProto
    from verl_b200.models import preset
    from verl_b200.workers.actor.dp_actor import DataParallelPPOActor
    from verl_b200.workers.config import FSDPActorConfig
    from verl_b200.workers.engine.native import NativeEngine

    class C(dict):
        __getattr__ = dict.get

    import numpy as np

    cfg = preset(name)
    eng = NativeEngine(cfg, C(), C(lr=1e-3, clip_grad=1.0), device="cpu", seed=3).initialize()
    actor = DataParallelPPOActor(FSDPActorConfig(ppo_mini_batch_size=2, ppo_micro_batch_size_per_gpu=1, use_kl_loss=False), eng)
    g = torch.Generator().manual_seed(2)
    P, R, B = 12, 6, 2
    img_tok = cfg.image_token_id
    grids = [torch.tensor([[1, 4, 4]]), torch.tensor([[1, 2, 4]])]          # 4 and 2 placeholder tokens
    ids = torch.zeros(B, P + R, dtype=torch.long)
    mask = torch.zeros(B, P + R, dtype=torch.long)
    pos = torch.zeros(B, 4, P + R, dtype=torch.long)
    mm = []
    for i, grid in enumerate(grids):
        n_img = int(grid.prod()) // 4
        prompt = [5 + i, 2002] + [img_tok] * n_img + [9, 11, 13]
        resp = torch.randint(3, 1900, (R - i,), generator=g).tolist()
        seq = torch.tensor(prompt + resp)
        lo = P - len(prompt)
        ids[i, lo : lo + len(seq)] = seq
        mask[i, lo : lo + len(seq)] = 1
        p3, _ = get_rope_index(seq, grid, img_tok, 2)
        pos[i, 1:, lo : lo + len(seq)] = p3
        pos[i, 0, lo : lo + len(seq)] = torch.arange(len(seq))
        mm.append({"pixel_values": torch.randn(int(grid.prod()), 3 * 2 * 4 * 4, generator=g), "image_grid_thw": grid})
    data = DataProto.from_dict({"input_ids": ids, "attention_mask": mask, "position_ids": pos, "responses": ids[:, P:],
                                "response_mask": mask[:, P:]}, non_tensors={"multi_modal_inputs": np.array(mm, dtype=object)},
                               meta_info={"temperature": 1.0, "micro_batch_size": 1})
    lp, _ = actor.compute_log_prob(data, calculate_entropy=False)
    # direct forward, one sequence at a time
    from verl_b200.models import CausalLM, PackedBatch

    ref = CausalLM(cfg, dtype=torch.float32)
    ref.load_state_dict({k: v.float() for k, v in eng.zero.named_full_tensors()})
    for i in range(B):
        seq = ids[i][mask[i].bool()]
        p3 = pos[i, 1:][:, mask[i].bool()]
        with torch.no_grad():
            logits = ref(PackedBatch(seq, p3, torch.tensor([0, len(seq)], dtype=torch.int32), len(seq),
                                     pixel_values=mm[i]["pixel_values"], image_grid_thw=mm[i]["image_grid_thw"]))
        full_lp = torch.log_softmax(logits.float(), -1)[:-1].gather(1, seq[1:, None])[:, 0]
        n_resp = int(mask[i, P:].sum())
        torch.testing.assert_close(lp[i, :n_resp], full_lp[-n_resp:], atol=1e-4, rtol=1e-4)
    data.batch["old_log_probs"] = lp
    data.batch["advantages"] = torch.randn(B, R, generator=g)
    watch = ("visual.blocks.0.qkv", "visual.deepstack.0.fc1", "visual.pos_embed")
    before = {k: v.clone() for k, v in eng.zero.named_full_tensors() if k.startswith(watch)}
    with eng.train_mode():
        m = actor.update_policy(data)
    assert m["actor/grad_norm"][0] > 0
    after = {k: v for k, v in eng.zero.named_full_tensors() if k in before}
    assert all(not torch.equal(before[k], after[k]) for k in before), "a part of the vision tower did not train"


@pytest.mark.parametrize("name", ["tiny-qwen2-vl", "tiny-qwen3-vl", "tiny-qwen3-vl-moe"])
def test_vl_rollout_with_images_matches_full_recompute(name):
    """The paged engine with multimodal requests (vision tower at admission, placeholder embeddings and [3, T] positions
    in prefill, offset positions in burst decode) generates greedily what a full forward over the growing sequence
    predicts; two requests with the same text but other pixels do not share cached pages."""
    from verl_b200.models import CausalLM, PackedBatch, preset
    from verl_b200.rollout import NativeRolloutEngine, SamplingParams

    cfg = preset(name)
    model = CausalLM(cfg, dtype=torch.float32).init_weights(5)
    g = torch.Generator().manual_seed(3)
    grid = torch.tensor([[1, 4, 4]])
    tok = cfg.image_token_id
    prompt = [7, 2002] + [tok] * 4 + [9, 11, 13, 21, 22, 23, 24, 25, 26, 27, 28, 29]   # longer than one cache page
    reqs = [{"pixel_values": torch.randn(16, 96, generator=g), "image_grid_thw": grid} for _ in range(2)]
    eng = NativeRolloutEngine(model, max_num_seqs=4, max_model_len=64, max_num_batched_tokens=8, num_blocks=32, decode_burst=4)
    sp = SamplingParams(temperature=0.0, max_tokens=7, ignore_eos=True)
    for i, mm in enumerate(reqs):
        eng.add_request(f"r{i}", prompt, sp, multi_modal_inputs=mm)
    eng.add_request("text", [7, 9, 11, 13], sp)
    done = {}
    while eng.has_unfinished():
        for o in eng.step():
            done[o.request_id] = o.token_ids
    assert done["r0"] != done["r1"] or True  # different pixels usually give different continuations
    for i, mm in enumerate(reqs):
        seq = list(prompt)
        for _ in range(7):
            ids = torch.tensor(seq)
            pos3, _ = get_rope_index(ids, grid, tok, 2)
            with torch.no_grad():
                logits = model(PackedBatch(ids, pos3, torch.tensor([0, len(seq)], dtype=torch.int32), len(seq),
                                           pixel_values=mm["pixel_values"], image_grid_thw=grid))
            seq.append(int(logits[-1].argmax()))
        assert done[f"r{i}"] == seq[len(prompt):], (i, done[f"r{i}"], seq[len(prompt):])
    assert len(done["text"]) == 7


@pytest.mark.parametrize("name,frames,agent", [("tiny-qwen2-vl", 0, False), ("tiny-qwen3-vl", 0, False), ("tiny-qwen3-vl", 4, False),
                                               ("tiny-qwen2-vl", 0, True), ("tiny-qwen3-vl", 4, True)])
def test_grpo_on_a_vision_language_model_end_to_end(tmp_path, monkeypatch, name, frames, agent):
    """The trainer path for images: dataset rows with pixels and grids (native image -> patch processing, placeholder
    expansion, [4, S] position ids), rollout with images, multimodal RoPE positions of the generated sequences, actor
    and reference log-probs, one update. Two steps of GRPO on the tiny Qwen2-VL preset with synthetic images."""
    import json
    import math

    from verl_b200.trainer.main_ppo import run_ppo
    from verl_b200.utils.config import compose

    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    cfg = compose("ppo_trainer", [
        f"actor_rollout_ref.model.path=preset:{name}", "trainer.device=cpu", "trainer.n_gpus_per_node=1", "trainer.nnodes=1",
        "trainer.logger=[file]", "trainer.total_epochs=1", "trainer.total_training_steps=2", "trainer.val_before_train=false",
        f"trainer.default_local_dir={tmp_path}/ckpt", "trainer.save_freq=-1", "trainer.test_freq=-1",
        "trainer.project_name=cpu_e2e", "trainer.experiment_name=vl",
        "data.train_files=synthetic:16:6:10:16:1900:0", "data.synthetic_image_size=16", "data.val_files=null",
        f"data.synthetic_video_frames={frames}",  # > 0: a video (frame pairs, deepstack features at its tokens) per prompt
        "data.train_batch_size=4", "data.max_prompt_length=48", "data.max_response_length=12", "data.shuffle=false",
        "algorithm.adv_estimator=grpo", "actor_rollout_ref.rollout.n=2", "actor_rollout_ref.rollout.max_num_seqs=8",
        "actor_rollout_ref.rollout.max_num_batched_tokens=128", "actor_rollout_ref.rollout.tensor_model_parallel_size=1",
        "actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=4", "actor_rollout_ref.ref.log_prob_micro_batch_size_per_gpu=4",
        "actor_rollout_ref.actor.ppo_mini_batch_size=4", "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=4",
        "actor_rollout_ref.actor.use_kl_loss=true", "actor_rollout_ref.actor.optim.lr=1e-5"] + (
        # server mode: the single-turn agent loop sends the sample's patches and grids with its request (over HTTP)
        ["actor_rollout_ref.rollout.agent.use_agent_loop=true", "actor_rollout_ref.rollout.agent.num_workers=2",
         "data.return_raw_chat=true"] if agent else []))
    trainer = run_ppo(cfg, spmd=True)
    assert trainer.global_steps == 2 and bool(trainer.async_rollout_mode) == agent
    m = [json.loads(l) for l in open(tmp_path / "logs" / "cpu_e2e" / "vl.jsonl")][-1]["data"]
    for key in ("actor/pg_loss", "actor/grad_norm", "actor/kl_loss", "response_length/mean", "training/rollout_probs_diff_mean"):
        assert key in m and math.isfinite(m[key]), key
    assert m["actor/grad_norm"] > 0
    # the rollout engine (vision tower at admission, mrope in prefill / decode) and the trainer agree on the policy
    assert m["training/rollout_probs_diff_mean"] < 5e-3, m["training/rollout_probs_diff_mean"]


def test_qwen2_5_vl_tower_matches_hf():
    """Qwen2.5-VL: RMSNorm blocks with a gated SiLU MLP, attention inside windows except in the full-attention blocks,
    window-ordered patches restored after the merger. Logits of a sequence with two images (one of them with ragged
    edge windows) against ``transformers``; HF names round-trip."""
    pytest.importorskip("transformers")
    from transformers import Qwen2_5_VLConfig, Qwen2_5_VLForConditionalGeneration

    hf_cfg = Qwen2_5_VLConfig(
        text_config=dict(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]},
                         max_position_embeddings=512, tie_word_embeddings=False, rope_theta=10000.0),
        vision_config=dict(depth=3, hidden_size=32, out_hidden_size=64, intermediate_size=48, num_heads=2, in_channels=3,
                           patch_size=4, spatial_merge_size=2, temporal_patch_size=2, window_size=16,
                           fullatt_block_indexes=[1], hidden_act="silu"),
        image_token_id=500, video_token_id=501, vision_start_token_id=502, tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = Qwen2_5_VLForConditionalGeneration(hf_cfg).float().eval()
    cfg = ModelConfig.from_hf_dict(hf_cfg.to_dict())
    assert cfg.is_vl and cfg.model_type == "qwen2_5_vl"
    native = hf_to_native_state_dict(cfg, dict(hf.state_dict()))
    model = CausalLM(cfg, dtype=torch.float32)
    assert model.visual.c.variant == "qwen2_5_vl" and model.visual.c.embed_dim == 32 and model.visual.c.hidden_size == 64
    missing, unexpected = model.load_state_dict(native, strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    # image 1: 8 x 8 patches = 4 x 4 merged units = four 2 x 2 windows; image 2: 4 x 12 patches = 2 x 6 units: windows of
    # 2 x 2 units, three of them
    grid = torch.tensor([[1, 8, 8], [1, 4, 12]])
    g = torch.Generator().manual_seed(1)
    pixels = torch.randn(64 + 48, 3 * 2 * 4 * 4, generator=g)
    ids = torch.tensor([5, 502] + [500] * 16 + [7, 9, 502] + [500] * 12 + [11, 13])
    pos3, delta = get_rope_index(ids, grid, image_token_id=500, spatial_merge_size=2)
    with torch.no_grad():
        vis_ref = hf.model.visual(pixels, grid_thw=grid)
        vis_ref = vis_ref.pooler_output if hasattr(vis_ref, "pooler_output") else vis_ref
        torch.testing.assert_close(model.visual(pixels, grid), vis_ref, atol=2e-4, rtol=2e-4)
        mm = (ids == 500).int()[None]
        am = torch.ones(1, ids.numel(), dtype=torch.long)
        # the positions are passed explicitly: still images keep ONE temporal position (that of the image's start), the
        # rule of the model's release; the per-second scaling of video frames is not modelled here
        ref = hf(input_ids=ids[None], pixel_values=pixels, image_grid_thw=grid, attention_mask=am, mm_token_type_ids=mm,
                 position_ids=pos3[:, None])
        batch = PackedBatch(ids, pos3, torch.tensor([0, ids.numel()], dtype=torch.int32), ids.numel(), pixel_values=pixels,
                            image_grid_thw=grid)
        logits = model(batch)
    torch.testing.assert_close(logits, ref.logits[0], atol=3e-4, rtol=3e-4)
    back = native_to_hf_state_dict(cfg, native)
    ref_sd = dict(hf.state_dict())
    assert set(back) == set(ref_sd)
    for k in ref_sd:
        assert torch.equal(back[k], ref_sd[k]), k


def test_qwen3_vl_matches_hf():
    """Qwen3-VL: LayerNorm tower with an interpolated learned position table and full attention, deepstack features
    added to the hidden states of the image tokens after the first decoder layers, a Qwen3 decoder (QK-norm) with
    interleaved multimodal RoPE. Tower outputs, deepstack features and logits of a sequence with two images against
    ``transformers``; HF names round-trip."""
    pytest.importorskip("transformers")
    try:
        from transformers import Qwen3VLConfig, Qwen3VLForConditionalGeneration
    except ImportError:
        pytest.skip("this transformers version has no Qwen3-VL")

    hf_cfg = Qwen3VLConfig(
        text_config=dict(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=16, max_position_embeddings=512,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [3, 3, 2],
                                          "mrope_interleaved": True}),
        vision_config=dict(depth=3, hidden_size=32, out_hidden_size=64, intermediate_size=48, num_heads=2, in_channels=3,
                           patch_size=4, spatial_merge_size=2, temporal_patch_size=2, num_position_embeddings=36,
                           deepstack_visual_indexes=[0, 2], hidden_act="gelu_pytorch_tanh"),
        image_token_id=500, video_token_id=501, vision_start_token_id=502, tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = Qwen3VLForConditionalGeneration(hf_cfg).float().eval()
    with torch.no_grad():  # the defaults (zero biases, unit norms) would hide a swapped or dropped tensor
        for n, p in hf.named_parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))
    cfg = ModelConfig.from_hf_dict(hf_cfg.to_dict())
    assert cfg.is_vl and cfg.model_type == "qwen3_vl" and cfg.qk_norm and not cfg.attention_bias and cfg.mrope_interleaved
    assert cfg.mrope_section == [3, 3, 2] and cfg.rope_theta == 10000.0 and cfg.head_dim == 16
    native = hf_to_native_state_dict(cfg, dict(hf.state_dict()))
    model = CausalLM(cfg, dtype=torch.float32)
    assert model.visual.c.variant == "qwen3_vl" and model.num_deepstack == 2
    missing, unexpected = model.load_state_dict(native, strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    grid = torch.tensor([[1, 8, 8], [1, 4, 12]])
    g = torch.Generator().manual_seed(1)
    pixels = torch.randn(64 + 48, 3 * 2 * 4 * 4, generator=g)
    ids = torch.tensor([5, 502] + [500] * 16 + [7, 9, 502] + [500] * 12 + [11, 13])
    pos3, delta = get_rope_index(ids, grid, image_token_id=500, spatial_merge_size=2)
    with torch.no_grad():
        vis_ref = hf.model.visual(pixels, grid_thw=grid)
        out, taps = model.visual(pixels, grid, return_deepstack=True)
        torch.testing.assert_close(out, vis_ref.pooler_output, atol=2e-4, rtol=2e-4)
        assert len(taps) == 2
        for a, b in zip(taps, vis_ref.deepstack_features):
            torch.testing.assert_close(a, b, atol=2e-4, rtol=2e-4)
        mm = (ids == 500).int()[None]
        am = torch.ones(1, ids.numel(), dtype=torch.long)
        # positions computed by the model itself: the rule for still images is the one of get_rope_index
        ref = hf(input_ids=ids[None], pixel_values=pixels, image_grid_thw=grid, attention_mask=am, mm_token_type_ids=mm)
        ref_pos, ref_delta = hf.model.get_rope_index(ids[None], mm, image_grid_thw=grid, attention_mask=am)
        assert torch.equal(ref_pos[:, 0], pos3) and int(ref_delta) == delta
        batch = PackedBatch(ids, pos3, torch.tensor([0, ids.numel()], dtype=torch.int32), ids.numel(), pixel_values=pixels,
                            image_grid_thw=grid)
        logits = model(batch)
    torch.testing.assert_close(logits, ref.logits[0], atol=3e-4, rtol=3e-4)
    back = native_to_hf_state_dict(cfg, native)
    ref_sd = dict(hf.state_dict())
    assert set(back) == set(ref_sd), (set(back) ^ set(ref_sd))
    for k in ref_sd:
        assert torch.equal(back[k], ref_sd[k]), k
    # config round trip
    cfg2 = ModelConfig.from_hf_dict(cfg.to_hf_dict())
    assert cfg2.mrope_interleaved and cfg2.mrope_section == [3, 3, 2] and cfg2.extra["vision_config"]["deepstack_visual_indexes"] == [0, 2]


def test_qwen3_vl_moe_matches_hf():
    """Qwen3-VL with a mixture-of-experts decoder (experts stored as stacked tensors): logits of a sequence with an image
    against ``transformers``; names round-trip."""
    pytest.importorskip("transformers")
    try:
        from transformers import Qwen3VLMoeConfig, Qwen3VLMoeForConditionalGeneration
    except ImportError:
        pytest.skip("this transformers version has no Qwen3-VL-MoE")

    hf_cfg = Qwen3VLMoeConfig(
        text_config=dict(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=16, max_position_embeddings=512, num_experts=4, num_experts_per_tok=2,
                         moe_intermediate_size=32, decoder_sparse_step=1, mlp_only_layers=[], tie_word_embeddings=False,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [3, 3, 2],
                                          "mrope_interleaved": True}),
        vision_config=dict(depth=2, hidden_size=32, out_hidden_size=64, intermediate_size=48, num_heads=2, in_channels=3,
                           patch_size=4, spatial_merge_size=2, temporal_patch_size=2, num_position_embeddings=16,
                           deepstack_visual_indexes=[1], hidden_act="gelu_pytorch_tanh"),
        image_token_id=500, video_token_id=501, vision_start_token_id=502, tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = Qwen3VLMoeForConditionalGeneration(hf_cfg).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "experts" in n or n.endswith("gate.weight"):
                p.normal_(0.0, 0.05)  # the experts' tensors start uninitialised, the router at zero
    cfg = ModelConfig.from_hf_dict(hf_cfg.to_dict())
    assert cfg.is_vl and cfg.is_moe and cfg.model_type == "qwen3_vl_moe" and cfg.num_experts == 4 and cfg.mrope_interleaved
    native = hf_to_native_state_dict(cfg, dict(hf.state_dict()))
    model = CausalLM(cfg, dtype=torch.float32)
    missing, unexpected = model.load_state_dict(native, strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    grid = torch.tensor([[1, 4, 8]])
    pixels = torch.randn(32, 3 * 2 * 4 * 4, generator=torch.Generator().manual_seed(1))
    ids = torch.tensor([5, 502] + [500] * 8 + [7, 9, 11, 13])
    pos3, _ = get_rope_index(ids, grid, image_token_id=500, spatial_merge_size=2)
    with torch.no_grad():
        ref = hf(input_ids=ids[None], pixel_values=pixels, image_grid_thw=grid, attention_mask=torch.ones(1, ids.numel(), dtype=torch.long),
                 mm_token_type_ids=(ids == 500).int()[None])
        logits = model(PackedBatch(ids, pos3, torch.tensor([0, ids.numel()], dtype=torch.int32), ids.numel(), pixel_values=pixels,
                                   image_grid_thw=grid))
    torch.testing.assert_close(logits, ref.logits[0], atol=3e-4, rtol=3e-4)
    back = native_to_hf_state_dict(cfg, native)
    ref_sd = dict(hf.state_dict())
    assert set(back) == set(ref_sd), (set(back) ^ set(ref_sd))
    for k in ref_sd:
        assert torch.equal(back[k], ref_sd[k]), k
    assert ModelConfig.from_hf_dict(cfg.to_hf_dict()).num_experts == 4


def test_video_inputs_match_hf_and_the_rollout_engine():
    """A prompt with an image AND a video: the patches of frame pairs, the placeholder expansion and the multimodal
    RoPE positions (temporal axis advancing per frame group) give the logits of ``transformers``' Qwen2-VL; the rollout
    engine with the same inputs generates greedily what the full forward predicts."""
    pytest.importorskip("transformers")
    import numpy as np
    from transformers import Qwen2VLConfig, Qwen2VLForConditionalGeneration

    from verl_b200.rollout import NativeRolloutEngine, SamplingParams
    from verl_b200.utils.dataset.vision_utils import VLProcessor, videos_to_patches

    hf_cfg = Qwen2VLConfig(
        text_config=dict(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]},
                         max_position_embeddings=512, tie_word_embeddings=False, rope_theta=10000.0),
        vision_config=dict(depth=2, embed_dim=32, hidden_size=64, num_heads=2, mlp_ratio=2, in_channels=3, patch_size=4,
                           spatial_merge_size=2, temporal_patch_size=2),
        image_token_id=500, video_token_id=501, vision_start_token_id=502, tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = Qwen2VLForConditionalGeneration(hf_cfg).float().eval()
    cfg = ModelConfig.from_hf_dict(hf_cfg.to_dict())
    model = CausalLM(cfg, dtype=torch.float32)
    missing, unexpected = model.load_state_dict(hf_to_native_state_dict(cfg, dict(hf.state_dict())), strict=False)
    assert not missing and not unexpected
    rng = np.random.default_rng(0)
    video = rng.integers(0, 256, (5, 16, 24, 3), dtype=np.uint8)      # 5 frames -> 3 frame groups (the last frame repeated)
    image = rng.integers(0, 256, (16, 16, 3), dtype=np.uint8)
    pvv, vgrid = videos_to_patches([video], 4, 2, 2)
    assert vgrid.tolist() == [[3, 4, 6]] and pvv.shape == (72, 3 * 2 * 4 * 4)
    # frame group 1, first patch of its first merge block = pixels [0:4, 0:4] of frames 2 and 3
    from verl_b200.utils.dataset.vision_utils import _CLIP_MEAN, _CLIP_STD

    want = (torch.from_numpy(video[2:4, :4, :4].astype(np.float32) / 255.0) - torch.tensor(_CLIP_MEAN)) / torch.tensor(_CLIP_STD)
    torch.testing.assert_close(pvv[24].view(3, 2, 4, 4), want.permute(3, 0, 1, 2))
    proc = VLProcessor.from_model_config(cfg)
    assert proc.video_token_id == 501
    prompt = [5, 502, 500, 7, 502, 501, 9, 11]
    ids, mm, pos3 = proc(prompt, [image], [video])
    assert ids.count(500) == 4 and ids.count(501) == 18 and set(mm) == {"pixel_values", "image_grid_thw", "pixel_values_videos", "video_grid_thw"}
    ids_t = torch.tensor(ids)
    with torch.no_grad():
        mmt = torch.zeros(1, len(ids), dtype=torch.int32)
        mmt[0, ids_t == 500], mmt[0, ids_t == 501] = 1, 2
        ref = hf(input_ids=ids_t[None], pixel_values=mm["pixel_values"], image_grid_thw=mm["image_grid_thw"],
                 pixel_values_videos=mm["pixel_values_videos"], video_grid_thw=mm["video_grid_thw"],
                 attention_mask=torch.ones(1, len(ids), dtype=torch.long), mm_token_type_ids=mmt, position_ids=pos3[:, None])
        batch = PackedBatch(ids_t, pos3, torch.tensor([0, len(ids)], dtype=torch.int32), len(ids), pixel_values=mm["pixel_values"],
                            image_grid_thw=mm["image_grid_thw"], pixel_values_videos=mm["pixel_values_videos"],
                            video_grid_thw=mm["video_grid_thw"])
        logits = model(batch)
    torch.testing.assert_close(logits, ref.logits[0], atol=3e-4, rtol=3e-4)
    # temporal axis: the video's three frame groups sit at consecutive temporal positions
    vid_t = pos3[0][ids_t == 501]
    assert vid_t.unique().numel() == 3 and int(vid_t.max() - vid_t.min()) == 2

    eng = NativeRolloutEngine(model, max_num_seqs=2, max_model_len=64, max_num_batched_tokens=16, num_blocks=16, decode_burst=2)
    out = eng.generate([ids], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True), multi_modal_inputs=[mm])[0]
    seq = list(ids)
    for _ in range(5):
        t = torch.tensor(seq)
        p3, _ = get_rope_index(t, mm["image_grid_thw"], 500, 2, video_grid_thw=mm["video_grid_thw"], video_token_id=501)
        with torch.no_grad():
            lg = model(PackedBatch(t, p3, torch.tensor([0, len(seq)], dtype=torch.int32), len(seq), pixel_values=mm["pixel_values"],
                                   image_grid_thw=mm["image_grid_thw"], pixel_values_videos=mm["pixel_values_videos"],
                                   video_grid_thw=mm["video_grid_thw"]))
        lg[:, [500, 501]] = float("-inf")  # the engine never samples a placeholder id
        seq.append(int(lg[-1].argmax()))
    assert out.token_ids == seq[len(ids):], (out.token_ids, seq[len(ids):])
