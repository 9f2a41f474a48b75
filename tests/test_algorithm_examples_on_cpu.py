"""Every algorithm of examples/algorithms/run_algorithm.sh trains for a step on the tiny model with exactly the overrides
the script would pass (DRY_RUN prints them)."""
import json
import math
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPT = os.path.join(ROOT, "examples", "algorithms", "run_algorithm.sh")
ALGOS = ["rloo", "remax", "reinforce_plus_plus", "reinforce_plus_plus_baseline", "opo", "grpo_passk", "gpg", "otb", "gspo", "sapo",
         "gmpo", "cispo", "clip_cov", "kl_cov"]


@pytest.mark.parametrize("algo", ALGOS)
def test_algorithm_example_trains_a_step(tmp_path, monkeypatch, algo):
    from test_e2e_grpo_on_cpu import _overrides

    from verl_b200.trainer.main_ppo import run_ppo
    from verl_b200.utils.config import compose

    out = subprocess.run(["bash", SCRIPT], env={**os.environ, "ALGO": algo, "DRY_RUN": "1"}, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    algo_overrides = out.stdout.split()
    assert algo_overrides and all("=" in o for o in algo_overrides)
    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    base = _overrides(tmp_path, ["trainer.n_gpus_per_node=1", "trainer.total_training_steps=1", "trainer.save_freq=-1",
                                 f"trainer.experiment_name={algo}", "data.max_response_length=16", "data.train_batch_size=4",
                                 "actor_rollout_ref.actor.ppo_mini_batch_size=4"])
    trainer = run_ppo(compose("ppo_trainer", base + algo_overrides), spmd=True)
    assert trainer.global_steps == 1
    m = [json.loads(l) for l in open(tmp_path / "logs" / "cpu_e2e" / f"{algo}.jsonl")][-1]["data"]
    assert math.isfinite(m["actor/pg_loss"]) and math.isfinite(m["actor/grad_norm"])


def test_unknown_algorithm_is_refused():
    out = subprocess.run(["bash", SCRIPT], env={**os.environ, "ALGO": "nope", "DRY_RUN": "1"}, capture_output=True, text=True)
    assert out.returncode == 2 and "unknown ALGO" in out.stderr


def test_sum_pi_squared_matches_dense_softmax():
    """``actor.calculate_sum_pi_squared``: compute_log_prob's third result equals sum_v softmax(logits / T)_v^2 of a plain
    forward, at the response tokens (dynamic batching on, so the rows come back in the original order)."""
    import torch

    from verl_b200 import DataProto
    from verl_b200.models import CausalLM, PackedBatch, preset
    from verl_b200.workers.actor.dp_actor import DataParallelPPOActor
    from verl_b200.workers.config import FSDPActorConfig
    from verl_b200.workers.engine.native import NativeEngine

    class C(dict):
        __getattr__ = dict.get

    cfg = preset("tiny-qwen2")
    eng = NativeEngine(cfg, C(), C(lr=1e-3), device="cpu", seed=2).initialize()
    actor = DataParallelPPOActor(FSDPActorConfig(ppo_mini_batch_size=4, calculate_sum_pi_squared=True), eng)
    g = torch.Generator().manual_seed(0)
    B, P, R, T = 4, 5, 7, 0.8
    ids = torch.randint(3, 2000, (B, P + R), generator=g)
    mask = torch.ones(B, P + R, dtype=torch.long)
    mask[0, :3] = 0
    mask[2, -4:] = 0
    pos = (mask.cumsum(-1) - 1).clamp(min=0)
    data = DataProto.from_dict({"input_ids": ids, "attention_mask": mask, "position_ids": pos, "responses": ids[:, P:]},
                               meta_info={"temperature": T, "use_dynamic_bsz": True, "max_token_len": 24})
    with eng.eval_mode():
        lp, _ = actor.compute_log_prob(data)
    spp = actor.last_sum_pi_squared
    assert spp.shape == (B, R)
    ref = CausalLM(cfg, dtype=torch.float32)
    ref.load_state_dict({k: v.float() for k, v in eng.zero.named_full_tensors()})
    for i in range(B):
        seq = ids[i][mask[i].bool()]
        with torch.no_grad():
            logits = ref(PackedBatch(seq, torch.arange(len(seq)), torch.tensor([0, len(seq)], dtype=torch.int32), len(seq)))
        p = torch.softmax(logits.float() / T, -1)
        n = int(mask[i, P:].sum())
        want = (p * p).sum(-1)[-n - 1 : -1]
        torch.testing.assert_close(spp[i, :n], want, atol=1e-5, rtol=1e-4)
        assert bool((spp[i, n:] == 0).all())
    with eng.train_mode():  # the update does not ask for it
        assert actor._want_spp is False


@pytest.mark.parametrize("mode", ["token_is", "seq_is", "token_rs", "bypass"])
def test_rollout_correction_example_modes_train_a_step(tmp_path, monkeypatch, mode):
    from test_e2e_grpo_on_cpu import _overrides

    from verl_b200.trainer.main_ppo import run_ppo
    from verl_b200.utils.config import compose

    script = os.path.join(ROOT, "examples", "rollout_correction", "run_qwen2_5-7b_rollout_correction.sh")
    out = subprocess.run(["bash", script], env={**os.environ, "MODE": mode, "DRY_RUN": "1"}, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    base = _overrides(tmp_path, ["trainer.n_gpus_per_node=1", "trainer.total_training_steps=1", "trainer.save_freq=-1",
                                 f"trainer.experiment_name={mode}", "data.max_response_length=16", "data.train_batch_size=4",
                                 "actor_rollout_ref.actor.ppo_mini_batch_size=4", "actor_rollout_ref.rollout.calculate_log_probs=true"])
    trainer = run_ppo(compose("ppo_trainer", base + out.stdout.split()), spmd=True)
    assert trainer.global_steps == 1
    m = [json.loads(l) for l in open(tmp_path / "logs" / "cpu_e2e" / f"{mode}.jsonl")][-1]["data"]
    assert math.isfinite(m["actor/pg_loss"]) and math.isfinite(m["actor/grad_norm"])
    if mode != "bypass":  # bypass: the rollout's log-probs ARE the old log-probs, there is no separate pass to compare with
        assert any(k.startswith("rollout_corr/") for k in m), sorted(m)[:40]
