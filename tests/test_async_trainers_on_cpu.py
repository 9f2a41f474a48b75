"""One-step-off and fully asynchronous trainers on CPU (tiny model, in-process worker group)."""

import math
import threading
import time

from verl_b200.utils.config import compose

from test_e2e_grpo_on_cpu import _overrides


def test_message_queue_staleness_and_backpressure():
    from verl_b200.experimental.fully_async_policy import MessageQueue

    q = MessageQueue(max_queue_size=4, max_staleness=1)
    for i in range(6):
        q.put_sample(i, param_version=0)
    st = q.get_statistics()
    assert st["queue_size"] == 4 and st["dropped_samples"] == 2
    got = q.get_samples(2)
    assert [s.data for s in got] == [2, 3]
    q.update_param_version(2)  # remaining version-0 samples are now 2 versions old: dropped
    assert q.get_queue_size() == 0 and q.get_statistics()["dropped_stale"] == 2
    assert q.get_samples(1, timeout=0.05) is None
    t = threading.Thread(target=lambda: (time.sleep(0.05), q.put_sample("x", 2)))
    t.start()
    assert q.get_samples(1, timeout=2.0)[0].data == "x"
    t.join()
    q.close()
    assert q.get_samples(1) is None


def test_metrics_aggregator_rules():
    from verl_b200.experimental.fully_async_policy import MetricsAggregator

    a = MetricsAggregator()
    a.add_step_metrics({"timing_s/gen": 1.0, "actor/pg_loss": 2.0, "response_length/max": 5.0, "training/global_step": 1})
    a.add_step_metrics({"timing_s/gen": 3.0, "actor/pg_loss": 4.0, "response_length/max": 9.0, "training/global_step": 2})
    m = a.get_aggregated_metrics()
    assert m["timing_s/gen"] == 4.0 and m["actor/pg_loss"] == 3.0 and m["response_length/max"] == 9.0
    assert m["training/global_step"] == 2


def test_one_step_off_trainer(tmp_path, monkeypatch):
    from verl_b200.experimental.one_step_off_policy import OneStepOffRayTrainer
    from verl_b200.trainer.main_ppo import run_ppo

    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    cfg = compose("ppo_trainer", _overrides(tmp_path, ["trainer.n_gpus_per_node=1", "trainer.total_training_steps=3",
                                                       "trainer.save_freq=-1"]))
    t = run_ppo(cfg, spmd=True, trainer_cls=OneStepOffRayTrainer)
    assert t.global_steps == 3


def test_fully_async_pipeline(tmp_path, monkeypatch):
    from verl_b200.experimental.fully_async_policy import run_fully_async
    from verl_b200.trainer.main_ppo import run_ppo

    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    cfg = compose("ppo_trainer", _overrides(tmp_path, ["trainer.n_gpus_per_node=1", "trainer.save_freq=-1"]))
    trainer = run_ppo(cfg, spmd=True, run_fit=False)
    try:
        out = run_fully_async(trainer, total_train_steps=3, required_samples=4, max_staleness=8, step_timeout=300)
    finally:
        trainer.shutdown()
    assert len(out) == 3
    for m in out:
        assert math.isfinite(m["actor/pg_loss"]) and "fully_async/staleness_mean" in m and "timing_s/param_sync" in m
    assert out[-1]["fully_async/param_version"] >= 2


def test_fully_async_pipeline_with_partial_rollouts(tmp_path, monkeypatch):
    """Prompt groups stream through the agent-loop manager; every parameter update aborts the generations in flight
    and they are resumed afterwards. Training steps complete and (with long responses on a slow CPU engine) some
    generations are indeed cut and continued."""
    from verl_b200.experimental.fully_async_policy import run_fully_async
    from verl_b200.trainer.main_ppo import run_ppo

    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    cfg = compose("ppo_trainer", _overrides(tmp_path, ["trainer.n_gpus_per_node=1", "trainer.save_freq=-1",
                                                       "actor_rollout_ref.rollout.free_cache_engine=false",
                                                       "actor_rollout_ref.rollout.agent.num_workers=2",
                                                       "data.max_response_length=24", "actor_rollout_ref.rollout.n=2"]))
    trainer = run_ppo(cfg, spmd=True, run_fit=False)
    try:
        out = run_fully_async(trainer, total_train_steps=3, required_samples=2, max_staleness=16, step_timeout=300,
                              partial_rollout=True, max_concurrent_groups=4)
        r = trainer.fully_async_rollouter
    finally:
        trainer.shutdown()
    assert len(out) == 3 and r.error is None and r.produced_groups >= 6
    for m in out:
        assert math.isfinite(m["actor/pg_loss"]) and "fully_async/staleness_mean" in m and "timing_s/param_sync" in m
    assert out[-1]["fully_async/param_version"] >= 2
    print("cancelled generations:", r.cancelled_generations)
