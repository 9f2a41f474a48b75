"""LoRA on the native engine: frozen base, trained adapters, merged export, checkpoint, and a GRPO run (CPU)."""

import os
import subprocess
import sys

import torch

from verl_b200.models import preset
from verl_b200.models.transformer import PackedBatch


class C(dict):
    __getattr__ = dict.get


def _batch(cfg, seed=0):
    lens = [9, 14, 6]
    ids = torch.randint(3, cfg.vocab_size, (sum(lens),), generator=torch.Generator().manual_seed(seed))
    cu = torch.tensor([0, 9, 23, 29], dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens])
    return PackedBatch(ids, pos, cu, max(lens)), torch.arange(ids.numel()), torch.roll(ids, -1)


def test_lora_trains_adapters_only_and_exports_merged_weights(tmp_path):
    from verl_b200.models.lora import lora_named_parameters
    from verl_b200.workers.engine.native import NativeEngine

    cfg = preset("tiny-qwen2")
    lora = {"rank": 8, "alpha": 16, "target_modules": ["q_proj", "down_proj"]}
    eng = NativeEngine(cfg, C(), C(lr=5e-2, clip_grad=10.0, weight_decay=0.0), device="cpu", seed=2, lora=lora).initialize()
    assert eng.zero.master is None and not eng.zero.trainable  # no optimizer state for the base
    assert sorted(eng.model.lora_modules) == sorted(f"layers.{i}.{m}" for i in range(cfg.num_hidden_layers)
                                                    for m in ("self_attn.qkv_proj", "mlp.down_proj"))
    assert not any("lora" in n for n, _ in eng.model.named_parameters())
    base0 = eng.zero.shard16.clone()
    batch, rows, labels = _batch(cfg)
    with eng.eval_mode():
        lp0, _ = eng.forward_logprob(batch, rows, labels, 1.0)
        with eng.disable_adapter():
            lp_ref0, _ = eng.forward_logprob(batch, rows, labels, 1.0)
    assert torch.allclose(lp0, lp_ref0)  # B starts at zero
    losses = []
    for _ in range(8):
        with eng.train_mode():
            eng.optimizer_zero_grad()
            lp, _ = eng.forward_logprob(batch, rows, labels, 1.0)
            loss = -lp.mean()
            loss.backward()
            gn = eng.optimizer_step()
        losses.append(float(loss))
        assert float(gn) > 0
    assert losses[-1] < losses[0] - 0.05, losses
    assert torch.equal(eng.zero.shard16, base0)  # base untouched
    assert any(float(p.abs().sum()) > 0 for n, p in lora_named_parameters(eng.model) if n.endswith("lora_B"))
    with eng.eval_mode():
        lp1, _ = eng.forward_logprob(batch, rows, labels, 1.0)
        with eng.disable_adapter():
            lp_ref1, _ = eng.forward_logprob(batch, rows, labels, 1.0)
    assert torch.allclose(lp_ref1, lp_ref0) and not torch.allclose(lp1, lp0)

    # merged export: a plain model loaded from it reproduces the adapted log-probs
    merged = eng.full_state_dict(dtype=torch.float32)
    plain = NativeEngine(cfg, C(), None, device="cpu", seed=5, trainable=False, state_dict=merged).initialize()
    with plain.eval_mode():
        lp_m, _ = plain.forward_logprob(batch, rows, labels, 1.0)
    torch.testing.assert_close(lp_m, lp1, atol=1e-4, rtol=1e-4)

    # checkpoint round trip (adapter + its optimizer), PEFT-style adapter files
    eng.save_checkpoint(str(tmp_path / "ck"), global_step=3)
    assert (tmp_path / "ck" / "lora_adapter" / "adapter_config.json").exists()
    from safetensors.torch import load_file

    ad = load_file(str(tmp_path / "ck" / "lora_adapter" / "adapter_model.safetensors"))
    q = cfg.num_attention_heads * cfg.head_dim
    assert ad["base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight"].shape == (q, 8)
    assert "base_model.model.model.layers.0.mlp.down_proj.lora_A.weight" in ad
    eng2 = NativeEngine(cfg, C(), C(lr=5e-2), device="cpu", seed=2, lora=lora).initialize()
    eng2.load_checkpoint(str(tmp_path / "ck"))
    with eng2.eval_mode():
        lp2, _ = eng2.forward_logprob(batch, rows, labels, 1.0)
    torch.testing.assert_close(lp2, lp1)
    assert eng2.step_count == eng.step_count


def test_lora_grpo_end_to_end(tmp_path, monkeypatch):
    """Two GRPO steps through the trainer with lora_rank > 0 on 2 worker processes: reference log-probs come from the
    actor with adapters off (no reference engine), the rollout copies receive merged weights, adapter files are saved."""
    import json
    import math

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from test_e2e_grpo_on_cpu import _overrides

    from verl_b200.trainer.main_ppo import run_ppo
    from verl_b200.utils.config import compose

    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    cfg = compose("ppo_trainer", _overrides(tmp_path, ["actor_rollout_ref.model.lora_rank=8", "actor_rollout_ref.model.lora_alpha=16",
                                                       "actor_rollout_ref.actor.optim.lr=1e-3", "trainer.experiment_name=lora",
                                                       "data.max_response_length=24", "actor_rollout_ref.rollout.n=2"]))
    trainer = run_ppo(cfg, spmd=False)
    assert trainer.global_steps == 2
    rows = [json.loads(l) for l in open(tmp_path / "logs" / "cpu_e2e" / "lora.jsonl")]
    m = rows[-1]["data"]
    for key in ("actor/pg_loss", "actor/grad_norm", "actor/kl_loss", "timing_s/ref"):
        assert key in m and math.isfinite(m[key]), key
    assert m["actor/grad_norm"] > 0
    step_dir = tmp_path / "ckpt" / "global_step_2" / "actor"
    assert (step_dir / "lora_adapter" / "adapter_model.safetensors").exists()
    assert (step_dir / "lora_train_state.pt").exists() and not (step_dir / "optim_world_size_2_rank_0.pt").exists()


def test_sft_with_lora(tmp_path):
    """SFT with model.lora_rank > 0: the loss goes down while only the adapters change."""
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from test_sft_on_cpu import _config

    from verl_b200.trainer.sft_trainer import SFTTrainer
    from verl_b200.utils.dataset.sft_dataset import sft_collate_fn
    from verl_b200.utils.tokenizer import IntTokenizer

    cfg = _config(tmp_path, **{"model.lora_rank": 8, "optim.lr": "2e-2"})
    tr = SFTTrainer(cfg, tokenizer=IntTokenizer(256))
    assert tr.engine._lora_params and tr.engine.zero.master is None
    base0 = tr.engine.zero.shard16.clone()
    losses = []
    for step, (_, idx) in enumerate(tr._batches(0)):
        losses.append(tr.train_step(sft_collate_fn([tr.train_dataset[i] for i in idx]))["train/loss"])
        tr.global_step += 1
        if step == 5:
            break
    assert losses[-1] < losses[0] and torch.equal(tr.engine.zero.shard16, base0)


def test_lora_single_process_rollout_copy_gets_merged_weights(tmp_path, monkeypatch):
    """World size 1: the rollout model is a separate copy under LoRA (it would share the actor's tensors otherwise);
    after a step it holds base + delta."""
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from test_e2e_grpo_on_cpu import _overrides

    from verl_b200.models.lora import lora_delta
    from verl_b200.trainer.main_ppo import run_ppo
    from verl_b200.utils.config import compose

    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    cfg = compose("ppo_trainer", _overrides(tmp_path, ["actor_rollout_ref.model.lora_rank=8", "actor_rollout_ref.actor.optim.lr=1e-2",
                                                       "trainer.n_gpus_per_node=1", "trainer.save_freq=-1",
                                                       "data.max_response_length=16", "actor_rollout_ref.rollout.n=2"]))
    trainer = run_ppo(cfg, spmd=True)
    w = trainer.actor_rollout_wg.worker.worker_dict["actor_rollout"]
    assert w.ref_engine is None and w.rollout_model is not w.actor_engine.model
    name = w.actor_engine.model.lora_modules[0]
    base_w = dict(w.actor_engine.zero.named_full_tensors())[name + ".weight"].float()
    roll_w = dict(w.rollout_model.named_parameters())[name + ".weight"].float()
    delta = lora_delta(dict(w.actor_engine.model.named_modules())[name])
    assert float(delta.abs().sum()) > 0
    torch.testing.assert_close(roll_w, base_w + delta, atol=1e-5, rtol=1e-5)
