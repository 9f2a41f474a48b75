"""Config composition, sequence-length balancing, the C++ continuous-batching scheduler, metrics, reward scores."""

import math

import numpy as np
import pytest
import torch

from verl_b200.utils.config import compose, select, to_config


def test_compose_defaults_overrides_interpolation():
    cfg = compose("ppo_trainer", ["actor_rollout_ref.actor.optim.lr=3e-6", "trainer.total_epochs=7", "+extra.key=5",
                                  "data.train_batch_size=64"])
    assert cfg.actor_rollout_ref.actor.optim.lr == pytest.approx(3e-6) and cfg.trainer.total_epochs == 7
    assert cfg.extra.key == 5 and cfg.data.train_batch_size == 64
    # interpolations of the reference tree resolve
    assert cfg.actor_rollout_ref.rollout.prompt_length == cfg.data.max_prompt_length
    assert cfg.critic.ppo_epochs == cfg.actor_rollout_ref.actor.ppo_epochs
    assert select(cfg, "actor_rollout_ref.actor.clip_ratio") == pytest.approx(0.2)
    assert select(cfg, "does.not.exist", "dflt") == "dflt"
    with pytest.raises(Exception):
        compose("ppo_trainer", ["nonexistent_group.key=1"])  # new keys need the + prefix


def test_validate_config_catches_bad_batch_sizes():
    from verl_b200.utils.config import validate_config

    cfg = compose("ppo_trainer", ["trainer.n_gpus_per_node=4", "data.train_batch_size=6", "actor_rollout_ref.rollout.n=1",
                                  "actor_rollout_ref.actor.ppo_mini_batch_size=6",
                                  "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=1",
                                  "actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=1"])
    with pytest.raises((AssertionError, ValueError)):
        validate_config(cfg, use_reference_policy=False, use_critic=False)  # 6 samples do not split over 4 GPUs


def test_karmarkar_karp_balances_and_keeps_all_items():
    from verl_b200.utils.seqlen_balancing import get_seqlen_balanced_partitions, log_seqlen_unbalance

    g = np.random.default_rng(0)
    lens = g.integers(10, 2000, size=64).tolist()
    for equal in (True, False):
        parts = get_seqlen_balanced_partitions(lens, 8, equal_size=equal)
        assert sorted(i for p in parts for i in p) == list(range(64))
        if equal:
            assert all(len(p) == 8 for p in parts)
        sums = [sum(lens[i] for i in p) for p in parts]
        assert max(sums) - min(sums) <= 0.1 * np.mean(sums)
    m = log_seqlen_unbalance(lens, parts, "x")
    assert m["x/balanced_max"] <= m["x/max"]


def test_rearrange_micro_batches_token_budget():
    from verl_b200.utils.seqlen_balancing import rearrange_micro_batches
    from verl_b200.utils.tensordict_lite import TensorDict

    g = torch.Generator().manual_seed(0)
    lens = torch.randint(5, 60, (16,), generator=g)
    mask = (torch.arange(64)[None, :] < lens[:, None]).long()
    td = TensorDict({"attention_mask": mask, "input_ids": torch.zeros(16, 64, dtype=torch.long)}, batch_size=[16])
    micro, idx = rearrange_micro_batches(td, max_token_len=128)
    assert sorted(i for p in idx for i in p) == list(range(16))
    for mb in micro:
        assert int(mb["attention_mask"].sum()) <= 128


def test_scheduler_continuous_batching_prefix_cache_and_preemption():
    from verl_b200.rollout.engine import Scheduler

    sc = Scheduler(num_blocks=24, block_size=4, max_num_seqs=4, max_batched_tokens=16, max_model_len=40)
    prompt = list(range(100, 110))
    for sid in range(3):
        sc.add(sid, prompt, 6)  # same prompt: later sequences reuse the first one's full blocks
    produced = {0: 0, 1: 0, 2: 0}
    done_all = set()
    for step in range(200):
        n, _ = sc.step()
        if n == 0:
            if len(done_all) == 3:
                break
            continue
        assert int(sc.seq_ntok[:n].sum()) <= 16
        toks = np.full(n, 7, np.int64)
        done = sc.commit(toks, np.zeros(n, np.int32)).copy()
        for i in range(n):
            sid = int(sc.seq_ids[i])
            if sc.seq_prefill[i] != 2:
                produced[sid] += 1
            if done[i]:
                done_all.add(sid)
    assert done_all == {0, 1, 2}
    st = sc.stats()
    assert st["prefix_hits"] > 0 and st["running"] == 0 and st["waiting"] == 0
    for sid in range(3):
        out = sc.output(sid, 16)
        assert len(out) == 6 and all(t == 7 for t in out)
    # a pool too small for everyone at once forces preemption but every request still finishes
    sc2 = Scheduler(num_blocks=9, block_size=4, max_num_seqs=4, max_batched_tokens=64, max_model_len=32, prefix_caching=False)
    for sid in range(3):
        sc2.add(sid, list(range(200 + 16 * sid, 200 + 16 * sid + 12)), 10)
    fin = set()
    for _ in range(500):
        n, _ = sc2.step()
        if n == 0 and len(fin) == 3:
            break
        if n:
            done = sc2.commit(np.full(n, 9, np.int64), np.zeros(n, np.int32)).copy()
            fin.update(int(sc2.seq_ids[i]) for i in range(n) if done[i])
    assert fin == {0, 1, 2} and sc2.stats()["preempted"] > 0


def test_data_and_throughput_metrics():
    from verl_b200.protocol import DataProto
    from verl_b200.trainer.ppo.metric_utils import (bootstrap_metric, compute_data_metrics, compute_throughout_metrics,
                                                    compute_timing_metrics, process_validation_metrics, reduce_metrics)

    B, P, R = 4, 3, 5
    mask = torch.ones(B, P + R, dtype=torch.long)
    mask[0, -2:] = 0
    batch = DataProto.from_dict(tensors={
        "prompts": torch.ones(B, P, dtype=torch.long), "responses": torch.ones(B, R, dtype=torch.long), "attention_mask": mask,
        "response_mask": mask[:, P:], "token_level_scores": torch.rand(B, R), "token_level_rewards": torch.rand(B, R),
        "advantages": torch.randn(B, R), "returns": torch.randn(B, R)})
    batch.meta_info["global_token_num"] = mask.sum(-1).tolist()
    m = compute_data_metrics(batch, use_critic=False)
    assert m["response_length/max"] == 5 and m["response_length/min"] == 3 and m["prompt_length/mean"] == 3
    t = compute_timing_metrics(batch, {"gen": 2.0, "update_actor": 1.0})
    assert t["timing_s/gen"] == 2.0 and "timing_per_token_ms/gen" in t
    th = compute_throughout_metrics(batch, {"step": 2.0}, n_gpus=2)
    assert th["perf/throughput"] == pytest.approx(int(mask.sum()) / 2.0 / 2)
    assert reduce_metrics({"a": [1.0, 3.0]})["a"] == 2.0
    (mean, std), = bootstrap_metric([1.0, 2.0, 3.0, 4.0], 2, [np.mean], n_bootstrap=200, seed=1)
    assert 2.0 < mean < 3.0 and std > 0
    val = process_validation_metrics(["src"] * 4, ["u1", "u1", "u2", "u2"], {"score": [1.0, 0.0, 1.0, 1.0]})
    assert val["src"]["score"]["mean@2"] == pytest.approx(0.75)


def test_reward_scores_rule_based():
    from verl_b200.utils.reward_score import default_compute_score, gsm8k, math_reward

    assert gsm8k.compute_score("so the answer is #### 42", "42") == 1.0
    assert gsm8k.compute_score("the answer is 42", "42") == 0.0
    assert math_reward.compute_score("thus \\\\boxed{\\\\frac{1}{2}}".replace("\\\\", "\\"), "\\frac{1}{2}") == 1.0
    assert default_compute_score("openai/gsm8k", "#### 7", "7") == 1.0
    r = default_compute_score("math_dapo", "Answer: 12", "12")
    assert (r["score"] if isinstance(r, dict) else r) > 0
    with pytest.raises(NotImplementedError):
        default_compute_score("unknown/source", "x", "y")
