"""End-to-end GRPO plumbing on CPU: tiny Qwen2-architecture policy, 2 worker processes over gloo, fp32.

Batch of 8 prompts x n=4 samples, 64-token prompts from [16, 2048), up to 64 response tokens, EOS id 2,
reward = fraction of even response ids, GRPO advantage, clip 0.2, KL-loss coefficient 0.001, AdamW lr 1e-6.
"""
import math
import os

import pytest

from verl_b200.utils.config import compose


def _overrides(tmp, extra=()):
    return [
        "actor_rollout_ref.model.path=preset:tiny-qwen2", "trainer.device=cpu", "trainer.n_gpus_per_node=2", "trainer.nnodes=1",
        "trainer.logger=[file]", "trainer.total_epochs=1", "trainer.total_training_steps=2", "trainer.val_before_train=false",
        f"trainer.default_local_dir={tmp}/ckpt", "trainer.save_freq=2", "trainer.test_freq=-1",
        "trainer.project_name=cpu_e2e", "trainer.experiment_name=grpo",
        "data.train_files=synthetic:32:64:64:16:2048:0", "data.val_files=null", "data.train_batch_size=8",
        "data.max_prompt_length=64", "data.max_response_length=64", "data.shuffle=false",
        "algorithm.adv_estimator=grpo", "algorithm.kl_ctrl.kl_coef=0.001",
        "actor_rollout_ref.rollout.n=4", "actor_rollout_ref.rollout.temperature=1.0", "actor_rollout_ref.rollout.max_num_seqs=16",
        "actor_rollout_ref.rollout.max_num_batched_tokens=256", "actor_rollout_ref.rollout.tensor_model_parallel_size=1",
        "actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=8", "actor_rollout_ref.ref.log_prob_micro_batch_size_per_gpu=8",
        "actor_rollout_ref.actor.ppo_mini_batch_size=8", "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=8",
        "actor_rollout_ref.actor.use_kl_loss=true", "actor_rollout_ref.actor.kl_loss_coef=0.001",
        "actor_rollout_ref.actor.clip_ratio=0.2", "actor_rollout_ref.actor.optim.lr=1e-6", "actor_rollout_ref.actor.ppo_epochs=1",
    ] + list(extra)


def test_grpo_two_cpu_workers(tmp_path, monkeypatch):
    import json

    from verl_b200.trainer.main_ppo import run_ppo

    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    cfg = compose("ppo_trainer", _overrides(tmp_path))
    trainer = run_ppo(cfg, spmd=False)
    assert trainer.global_steps == 2
    rows = [json.loads(l) for l in open(tmp_path / "logs" / "cpu_e2e" / "grpo.jsonl")]
    assert len(rows) == 2
    m = rows[-1]["data"]
    for key in ("actor/pg_loss", "actor/grad_norm", "actor/kl_loss", "actor/entropy", "critic/score/mean",
                "response_length/mean", "perf/throughput", "timing_s/gen", "timing_s/update_actor"):
        assert key in m and math.isfinite(m[key]), key
    assert 0.0 <= m["critic/score/mean"] <= 1.0
    assert m["actor/grad_norm"] > 0
    # checkpoint in the verl layout, one shard per rank
    step_dir = tmp_path / "ckpt" / "global_step_2"
    assert (tmp_path / "ckpt" / "latest_checkpointed_iteration.txt").read_text() == "2"
    for r in range(2):
        assert (step_dir / "actor" / f"model_world_size_2_rank_{r}.pt").exists()
        assert (step_dir / "actor" / f"optim_world_size_2_rank_{r}.pt").exists()
        assert (step_dir / "actor" / f"extra_state_world_size_2_rank_{r}.pt").exists()
    assert json.loads((step_dir / "actor" / "fsdp_config.json").read_text())["world_size"] == 2
    assert (step_dir / "actor" / "huggingface" / "config.json").exists()
    assert (step_dir / "data.pt").exists()


def test_ppo_with_critic_spmd_single_process(tmp_path, monkeypatch):
    """PPO + critic (GAE) through the in-process SPMD worker group, then resume from its checkpoint."""
    from verl_b200.trainer.main_ppo import run_ppo

    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    extra = ["algorithm.adv_estimator=gae", "actor_rollout_ref.rollout.n=1", "actor_rollout_ref.actor.use_kl_loss=false",
             "critic.model.path=preset:tiny-qwen2", "critic.ppo_micro_batch_size_per_gpu=8", "critic.optim.lr=1e-5",
             "trainer.n_gpus_per_node=1", "trainer.save_freq=1"]
    cfg = compose("ppo_trainer", _overrides(tmp_path, extra))
    t = run_ppo(cfg, spmd=True)
    assert t.global_steps == 2
    cfg2 = compose("ppo_trainer", _overrides(tmp_path, extra + ["trainer.total_training_steps=3"]))
    t2 = run_ppo(cfg2, spmd=True)
    assert t2.global_steps == 3  # resumed at 2, ran one more


@pytest.mark.parametrize("spmd", [True, False, "tool"])
def test_grpo_through_agent_loops(tmp_path, monkeypatch, spmd):
    """rollout.agent.use_agent_loop: rollouts go through the token-in / token-out server and the agent loops, in
    process (SPMD launch) and over HTTP to two worker processes."""
    import json

    from verl_b200.trainer.main_ppo import run_ppo

    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    extra = ["actor_rollout_ref.rollout.agent.use_agent_loop=true", "actor_rollout_ref.rollout.agent.num_workers=2",
             "trainer.save_freq=-1", "trainer.experiment_name=agent", "data.return_raw_chat=true",
             "data.max_response_length=24", "actor_rollout_ref.rollout.n=2"]
    if spmd == "tool":  # multi-turn configuration: the tool-calling state machine drives every sample
        extra = ["actor_rollout_ref.rollout.multi_turn.enable=true", "actor_rollout_ref.rollout.multi_turn.max_assistant_turns=2",
                 "actor_rollout_ref.rollout.agent.default_agent_loop=tool_agent"] + extra[1:]
    if spmd:
        extra.append("trainer.n_gpus_per_node=1")
    trainer = run_ppo(compose("ppo_trainer", _overrides(tmp_path, extra)), spmd=bool(spmd))
    assert trainer.async_rollout_mode and trainer.global_steps == 2
    m = [json.loads(l) for l in open(tmp_path / "logs" / "cpu_e2e" / "agent.jsonl")][-1]["data"]
    for key in ("actor/pg_loss", "actor/grad_norm", "response_length/mean", "agent_loop/generate_sequences/mean"):
        assert key in m and math.isfinite(m[key]), key
    assert m["response_length/mean"] > 0 and m["actor/grad_norm"] > 0


def test_task_runner_subclass_is_used(tmp_path, monkeypatch):
    """``run_ppo(config, task_runner_class=...)``: a subclass can swap a worker class."""
    from verl_b200.trainer.main_ppo import TaskRunner, run_ppo
    from verl_b200.trainer.ppo.utils import Role
    from verl_b200.workers.engine_workers import ActorRolloutRefWorker

    seen = []

    from verl_b200.single_controller.base.decorator import Dispatch, register

    class MyWorker(ActorRolloutRefWorker):
        @register(dispatch_mode=Dispatch.ONE_TO_ALL)  # an override is dispatched only if it is registered again
        def init_model(self):
            seen.append("init")
            return super().init_model()

    class MyRunner(TaskRunner):
        def add_actor_rollout_worker(self, config):
            super().add_actor_rollout_worker(config)
            self.role_worker_mapping[Role.ActorRollout] = MyWorker

    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    cfg = compose("ppo_trainer", _overrides(tmp_path, ["trainer.n_gpus_per_node=1", "trainer.save_freq=-1",
                                                       "trainer.total_training_steps=1", "data.max_response_length=8"]))
    t = run_ppo(cfg, spmd=True, task_runner_class=MyRunner)
    assert t.global_steps == 1 and seen == ["init"]


def test_dynamic_sampling_accumulates_over_generation_batches(tmp_path, monkeypatch):
    """algorithm.filter_groups: when a generation batch keeps only half of its prompt groups, the step trains after a
    second generation batch; the loader advances by one batch per generation batch (no rewinding) and the limit on
    generation batches raises."""
    import json

    from verl_b200.trainer.main_ppo import run_ppo
    from verl_b200.trainer.ppo.ray_trainer import RayPPOTrainer

    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    seen_prompts = []

    def keep_half(self, batch, metric_name):
        uids = list(dict.fromkeys(batch.non_tensor_batch["uid"]))
        seen_prompts.append(batch.batch["prompts"][:: int(self.config.actor_rollout_ref.rollout.n)].clone())
        keep = set(uids[: len(uids) // 2])
        return batch[[i for i, u in enumerate(batch.non_tensor_batch["uid"]) if u in keep]]

    monkeypatch.setattr(RayPPOTrainer, "_filter_groups", keep_half)
    extra = ["trainer.n_gpus_per_node=1", "trainer.save_freq=-1", "trainer.experiment_name=dyn",
             "+algorithm.filter_groups.enable=true", "+algorithm.filter_groups.metric=seq_reward",
             "+algorithm.filter_groups.max_num_gen_batches=0", "trainer.balance_batch=false"]
    t = run_ppo(compose("ppo_trainer", _overrides(tmp_path, extra)), spmd=True)
    assert t.global_steps == 2
    assert len(seen_prompts) == 4  # two generation batches per training step
    for a in range(4):
        for b in range(a + 1, 4):
            assert not (seen_prompts[a] == seen_prompts[b]).all(), "a generation batch reused earlier prompts"
    rows = [json.loads(l)["data"] for l in open(tmp_path / "logs" / "cpu_e2e" / "dyn.jsonl")]
    assert len(rows) == 2 and all(r["train/num_gen_batches"] == 2 for r in rows)
    extra[-2] = "+algorithm.filter_groups.max_num_gen_batches=1"
    extra[2] = "trainer.experiment_name=dyn_limit"
    with pytest.raises(ValueError, match="dynamic sampling"):
        run_ppo(compose("ppo_trainer", _overrides(tmp_path, extra)), spmd=True)


def test_grpo_with_tensor_parallel_rollout_replica(tmp_path, monkeypatch):
    """rollout.tensor_model_parallel_size=2 on two gloo workers: one replica sliced over both ranks (weights synced from
    the ZeRO shards into the TP layout), both ranks receive the same prompts, rank 0 reports."""
    import json

    from verl_b200.trainer.main_ppo import run_ppo

    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    extra = ["actor_rollout_ref.rollout.tensor_model_parallel_size=2", "trainer.save_freq=-1", "trainer.experiment_name=tp2",
             "actor_rollout_ref.rollout.max_num_seqs=32"]
    trainer = run_ppo(compose("ppo_trainer", _overrides(tmp_path, extra)), spmd=False)
    assert trainer.global_steps == 2
    m = [json.loads(l) for l in open(tmp_path / "logs" / "cpu_e2e" / "tp2.jsonl")][-1]["data"]
    for key in ("actor/pg_loss", "actor/grad_norm", "response_length/mean", "timing_s/gen"):
        assert key in m and math.isfinite(m[key]), key
    # rollout and training log-probs of the same tokens agree: the TP replica holds the trainer's weights
    assert abs(m.get("training/rollout_probs_diff_mean", 0.0)) < 1e-3


def test_agent_loops_over_a_tensor_parallel_replica(tmp_path, monkeypatch):
    """Server mode with rollout.tensor_model_parallel_size=2: the replica has ONE endpoint on its first rank; that
    rank's engine thread announces every request, abort, cache operation and step to the other rank's engine thread,
    which does the same to its slice of the model."""
    import json

    from verl_b200.trainer.main_ppo import run_ppo

    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    extra = ["actor_rollout_ref.rollout.tensor_model_parallel_size=2", "trainer.save_freq=-1", "trainer.experiment_name=tp2_agent",
             "actor_rollout_ref.rollout.max_num_seqs=32", "actor_rollout_ref.rollout.agent.use_agent_loop=true",
             "actor_rollout_ref.rollout.agent.num_workers=2", "data.return_raw_chat=true", "data.max_response_length=24",
             "actor_rollout_ref.rollout.n=2"]
    trainer = run_ppo(compose("ppo_trainer", _overrides(tmp_path, extra)), spmd=False)
    assert trainer.async_rollout_mode and trainer.global_steps == 2 and len(trainer._rollout_server_handles) == 1
    m = [json.loads(l) for l in open(tmp_path / "logs" / "cpu_e2e" / "tp2_agent.jsonl")][-1]["data"]
    # timing_s/resync is there only when the trainer waited for every worker's weight push: the servers take requests
    # outside the workers' command queues, so a push still running on one rank would race the next generation
    for key in ("actor/pg_loss", "actor/grad_norm", "response_length/mean", "agent_loop/generate_sequences/mean", "timing_s/resync"):
        assert key in m and math.isfinite(m[key]), key
    assert m["response_length/mean"] > 0 and abs(m.get("training/rollout_probs_diff_mean", 0.0)) < 1e-3


def test_async_reward_gives_the_same_step_as_the_synchronous_one(tmp_path, monkeypatch):
    """reward_model.launch_reward_fn_async: the rule-based reward runs on a host thread during the log-prob passes and is
    joined before the advantages (with batch balancing on, so rows are permuted before the reward starts)."""
    import json

    from verl_b200.trainer.main_ppo import run_ppo

    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    res = {}
    for flag in ("false", "true"):
        extra = ["trainer.n_gpus_per_node=1", "trainer.save_freq=-1", f"trainer.experiment_name=rw_{flag}",
                 f"reward_model.launch_reward_fn_async={flag}", "trainer.balance_batch=true", "trainer.total_training_steps=1"]
        run_ppo(compose("ppo_trainer", _overrides(tmp_path, extra)), spmd=True)
        res[flag] = [json.loads(l) for l in open(tmp_path / "logs" / "cpu_e2e" / f"rw_{flag}.jsonl")][-1]["data"]
    for key in ("critic/score/mean", "actor/pg_loss", "actor/grad_norm", "critic/advantages/mean"):
        assert abs(res["true"][key] - res["false"][key]) < 1e-6 * max(1.0, abs(res["false"][key])), key
    assert "timing_s/reward_wait" in res["true"]


def test_unservable_rollout_parallelism_is_an_error(tmp_path):
    from verl_b200.trainer.main_ppo import run_ppo

    with pytest.raises(Exception, match="tensor_model_parallel_size"):
        run_ppo(compose("ppo_trainer", _overrides(tmp_path, ["trainer.n_gpus_per_node=1", "trainer.save_freq=-1",
                                                             "actor_rollout_ref.rollout.tensor_model_parallel_size=2"])),
                spmd=True)
