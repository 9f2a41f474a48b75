"""Keeping layer activations instead of recomputing them gives the same step (2 gloo ranks, ZeRO-3)."""

import os
import subprocess
import sys


def test_kept_activations_match_recomputation():
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29950 + os.getpid() % 300), os.path.join(here, "_keep_act_worker.py")]
    env = {k: v for k, v in os.environ.items() if k != "VERL_B200_KEEP_ACTIVATION_LAYERS"}
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "KEEP_ACT_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])


def test_out_of_memory_in_a_training_forward_falls_back_to_recomputation(monkeypatch):
    """Single rank: an OOM raised while layers keep their activations is answered by one repeat of the forward with
    every layer recomputed (and the policy stays off); the step then matches a plain recomputing step."""
    import torch

    from verl_b200.models import preset
    from verl_b200.models.transformer import PackedBatch
    from verl_b200.parallel import zero as zmod
    from verl_b200.workers.engine.native import NativeEngine

    class C(dict):
        __getattr__ = dict.get

    cfg = preset("tiny-qwen2")
    ids = torch.randint(3, cfg.vocab_size, (20,), generator=torch.Generator().manual_seed(0))
    batch = PackedBatch(ids, torch.arange(20), torch.tensor([0, 20], dtype=torch.int32), 20)
    rows, labels = torch.arange(19), ids[1:]

    def step(eng):
        with eng.train_mode():
            eng.optimizer_zero_grad()
            lp, _ = eng.forward_logprob(batch, rows, labels, 1.0)
            (-lp.mean()).backward()
            return eng.zero.grad.clone()

    ref = step(NativeEngine(cfg, C(keep_activation_layers="0"), C(lr=1e-3), device="cpu", seed=1).initialize())
    eng = NativeEngine(cfg, C(keep_activation_layers=str(cfg.num_hidden_layers)), C(lr=1e-3), device="cpu", seed=1).initialize()
    calls = {"n": 0}
    real = zmod._UnitFnKeep.forward

    def boom(ctx, *a):
        calls["n"] += 1
        raise torch.cuda.OutOfMemoryError("fake")

    monkeypatch.setattr(zmod._UnitFnKeep, "forward", staticmethod(boom))
    got = step(eng)
    monkeypatch.setattr(zmod._UnitFnKeep, "forward", real)
    assert calls["n"] == 1 and eng._keep_cap == 0 and eng._layers_to_keep(20) == 0
    torch.testing.assert_close(got, ref)
