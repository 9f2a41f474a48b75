"""Failure detection without a GPU fault: lost ranks (host heartbeat / collective timeout), non-finite gradients,
damaged checkpoints, stale samples. Worker-process death is covered in test_single_controller_on_cpu.py."""

import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("mode", ["heartbeat", "timeout"])
def test_lost_rank_is_detected(mode):
    port = 29800 + (os.getpid() % 100) * 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "_rank_loss_worker.py"), mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=120)
    assert r.stdout.count("DETECTED " + mode) >= 1 and "NOT_DETECTED" not in r.stdout, (r.stdout[-2000:], r.stderr[-2000:])


def _engine(lr=1e-2):
    from verl_b200.models import preset
    from verl_b200.workers.engine.native import NativeEngine

    return NativeEngine(preset("tiny-qwen2"), None, {"lr": lr, "clip_grad": 1.0}, device="cpu", seed=1).initialize()


def test_non_finite_gradient_skips_the_update():
    eng = _engine()
    before = eng.zero.master.clone()
    with eng.train_mode():
        eng.optimizer_zero_grad()
        eng.zero.grad.fill_(1.0)
        eng.zero.grad[5] = float("nan")  # injected on the host
        gn = eng.optimizer_step()
    assert not torch.isfinite(torch.as_tensor(float(gn)))
    assert torch.equal(eng.zero.master, before)  # verl/workers/actor/dp_actor.py:410-412: skip, do not poison the weights
    with eng.train_mode():
        eng.optimizer_zero_grad()
        eng.zero.grad.fill_(1e-3)
        eng.optimizer_step()
    assert not torch.equal(eng.zero.master, before)


def test_damaged_checkpoint_shard_is_reported(tmp_path):
    eng = _engine()
    path = tmp_path / "ckpt"
    eng.save_checkpoint(str(path), global_step=1)
    shard = path / "model_world_size_1_rank_0.pt"
    data = shard.read_bytes()
    shard.write_bytes(data[: len(data) // 2])  # truncated file
    with pytest.raises(Exception):
        _engine().load_checkpoint(str(path))
    shard.unlink()
    with pytest.raises(Exception):
        _engine().load_checkpoint(str(path), load_contents=("model",))


def test_latest_checkpoint_tracker_ignores_missing_directories(tmp_path):
    from verl_b200.utils.checkpoint.checkpoint_manager import find_latest_ckpt_path, write_tracker

    root = tmp_path / "run"
    (root / "global_step_2").mkdir(parents=True)
    write_tracker(str(root), 5)  # tracker points at a step whose directory never got written
    assert find_latest_ckpt_path(str(root)) in (None, str(root / "global_step_2"))
    write_tracker(str(root), 2)
    assert find_latest_ckpt_path(str(root)) == str(root / "global_step_2")


def test_timeout_limit_and_esi_guard():
    import time

    from verl_b200.utils.checkpoint.checkpoint_manager import should_save_ckpt_esi
    from verl_b200.utils.py_functional import timeout_limit

    @timeout_limit(seconds=0.2)
    def slow():
        time.sleep(2)

    with pytest.raises(TimeoutError):
        slow()
    os.environ["MLP_CURRENT_CAPACITY_BLOCK_EXPIRATION_TIMESTAMP"] = str(int(time.time()) + 30)
    try:
        assert should_save_ckpt_esi(max_steps_duration=20.0, save_ckpt_duration=20.0)
    finally:
        del os.environ["MLP_CURRENT_CAPACITY_BLOCK_EXPIRATION_TIMESTAMP"]
    assert not should_save_ckpt_esi(max_steps_duration=20.0)
