"""OpenVLA-OFT policy on the native decoder: sequence assembly, parallel action decoding, log-prob recomputation,
gradients into every part, and the policy inside the pipelined environment loop (synthetic reach task)."""

import numpy as np
import torch


def _tiny(chunk=2, dim=2, proprio=0):
    from verl_b200.models import preset
    from verl_b200.models.openvla_oft import OpenVLAForActionPrediction, OpenVLAOFTConfig, ViTSpec

    cfg = OpenVLAOFTConfig(llm=preset("tiny-qwen2"), image_size=28, patch_size=14,
                           backbones=(ViTSpec(32, 3, 2, 2.0, True), ViTSpec(48, 3, 2, 2.0, False)), num_actions_chunk=chunk,
                           action_dim=dim, n_action_bins=16, proprio_dim=proprio,
                           norm_stats={"toy": {"action": {"q01": [-2.0] * dim, "q99": [2.0] * dim, "mask": [True] * (dim - 1) + [False]}}})
    return OpenVLAForActionPrediction(cfg, dtype=torch.float32, device="cpu").init_weights(3), cfg


def _inputs(B, lens, cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    L = max(lens)
    ids = torch.zeros(B, L, dtype=torch.long)
    mask = torch.zeros(B, L, dtype=torch.long)
    for b, n in enumerate(lens):
        ids[b, :n] = torch.randint(10, 1000, (n,), generator=g)
        ids[b, 0] = cfg.bos_token_id
        mask[b, :n] = 1
    pix = torch.randn(B, 3 * len(cfg.backbones), cfg.image_size, cfg.image_size, generator=g)
    return ids, mask, pix


def test_parallel_action_decoding_and_logprob_recomputation():
    model, cfg = _tiny(chunk=2, dim=3, proprio=4)
    ids, mask, pix = _inputs(3, [5, 9, 7], cfg)
    proprio = torch.randn(3, 4)
    out = model.generate_action(ids, mask, pix, proprio=proprio, temperature=0.7, generator=torch.Generator().manual_seed(1))
    A = cfg.num_actions_chunk * cfg.action_dim
    assert out["responses"].shape == (3, A) and out["actions"].shape == (3, 2, 3) and out["log_probs"].shape == (3, A)
    V = cfg.llm.vocab_size
    assert int(out["responses"].min()) >= V - cfg.n_action_bins and int(out["responses"].max()) < V
    # un-normalisation: masked dimensions map [-1, 1] -> [q01, q99], the last one passes through
    n = out["normalized_actions"]
    assert torch.allclose(out["actions"][..., 0], 2.0 * n[..., 0]) and torch.equal(out["actions"][..., -1], n[..., -1])
    # the actor recomputes exactly what the rollout stored (same temperature)
    lp, ent = model.action_log_probs(ids, mask, pix, out["responses"], proprio=proprio, temperature=0.7)
    assert torch.allclose(lp, out["log_probs"], atol=1e-5) and bool((ent > 0).all())
    # packing: a sample alone gives the same distribution as inside a batch of other lengths
    lp1, _ = model.action_log_probs(ids[1:2, :9], mask[1:2, :9], pix[1:2], out["responses"][1:2], proprio=proprio[1:2], temperature=0.7)
    assert torch.allclose(lp1, lp[1:2], atol=1e-5)
    # greedy decoding picks the most likely bin of every position
    greedy = model.generate_action(ids, mask, pix, proprio=proprio, do_sample=False)
    lp_g, _ = model.action_log_probs(ids, mask, pix, greedy["responses"], proprio=proprio)
    assert bool((lp_g >= model.action_log_probs(ids, mask, pix, out["responses"], proprio=proprio)[0] - 1e-6).all())


def test_gradients_reach_every_part_and_a_policy_gradient_step_raises_the_logprob():
    model, cfg = _tiny()
    ids, mask, pix = _inputs(4, [6, 6, 8, 5], cfg, seed=2)
    target = model.generate_action(ids, mask, pix, generator=torch.Generator().manual_seed(0))["responses"]
    opt = torch.optim.Adam(model.parameters(), lr=2e-3)
    first = None
    for _ in range(8):
        lp, _ = model.action_log_probs(ids, mask, pix, target)
        loss = -lp.mean()
        opt.zero_grad()
        loss.backward()
        if first is None:
            first = float(lp.detach().mean())
            for part in ("vision_backbone.towers.0.patch_embed.weight", "vision_backbone.towers.1.blocks.0.qkv.weight",
                         "projector.layers.0.weight", "language_model.layers.0.self_attn.qkv_proj.weight"):
                gnorm = dict(model.named_parameters())[part].grad
                assert gnorm is not None and float(gnorm.abs().sum()) > 0, part
            # the last ViT block does not feed the features (second-to-last block's output is used)
            assert dict(model.named_parameters())["vision_backbone.towers.0.blocks.2.qkv.weight"].grad is None
        opt.step()
    assert float(model.action_log_probs(ids, mask, pix, target)[0].mean()) > first + 0.05


def test_policy_drives_the_env_loop():
    from verl_b200.experimental.vla.env_loop import ActionTokenizer, EnvLoop
    from verl_b200.experimental.vla.envs.synthetic_env import SyntheticReachEnv
    from verl_b200.models.openvla_oft import OpenVLAPolicy

    model, cfg = _tiny(chunk=1, dim=2)
    policy = OpenVLAPolicy(model, tokenize=lambda s: [cfg.bos_token_id] + [10 + (ord(ch) % 500) for ch in s[:12]])
    loop = EnvLoop([lambda: SyntheticReachEnv(3, image_size=28, max_steps=4, seed=1), lambda: SyntheticReachEnv(3, image_size=28, max_steps=4, seed=2)],
                   policy, ActionTokenizer(n_bins=cfg.n_action_bins - 1), max_steps=4)
    trajs = loop.run()
    loop.close()
    data = loop.to_dataproto(trajs)
    assert data.batch["responses"].shape == (6, 4 * 2) and data.batch["rollout_log_probs"].shape == (6, 8)
    assert int(data.batch["responses"].max()) < cfg.n_action_bins and bool((data.batch["rollout_log_probs"] <= 0).all())
    assert np.isfinite(data.batch["token_level_scores"].numpy()).all()
