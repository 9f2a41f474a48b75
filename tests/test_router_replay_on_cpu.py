"""Router replay for mixture-of-experts policies: the experts recorded in compute_log_prob are the ones the update
routes to, also after the router's weights have moved."""
import torch

from verl_b200 import DataProto
from verl_b200.models import preset
from verl_b200.workers.actor.dp_actor import DataParallelPPOActor
from verl_b200.workers.config import FSDPActorConfig
from verl_b200.workers.engine.native import NativeEngine


class C(dict):
    __getattr__ = dict.get


def _batch(cfg, B=4, P=6, R=8, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(3, cfg.vocab_size - 8, (B, P + R), generator=g)
    mask = torch.ones(B, P + R, dtype=torch.long)
    mask[0, :2] = 0
    mask[1, -3:] = 0
    pos = (mask.cumsum(-1) - 1).clamp(min=0)
    return DataProto.from_dict({"input_ids": ids, "attention_mask": mask, "position_ids": pos, "responses": ids[:, P:],
                                "response_mask": mask[:, P:], "advantages": torch.randn(B, R, generator=g)},
                               meta_info={"temperature": 1.0, "micro_batch_size": 2})


def _actor(mode, seed=3, **kw):
    cfg = preset("tiny-qwen3-moe")
    eng = NativeEngine(cfg, C(), C(lr=5e-2, clip_grad=1.0), device="cpu", seed=seed).initialize()
    acfg = FSDPActorConfig(ppo_mini_batch_size=2, ppo_micro_batch_size_per_gpu=2, use_kl_loss=False, ppo_epochs=1,
                           router_replay={"mode": mode}, **kw)
    return cfg, eng, DataParallelPPOActor(acfg, eng)


def test_r2_records_in_log_prob_and_replays_in_the_update():
    cfg, eng, actor = _actor("R2")
    data = _batch(cfg)
    with eng.eval_mode():
        lp, _ = actor.compute_log_prob(data, calculate_entropy=False)
    rec = actor.last_routed_experts
    L, K = cfg.num_hidden_layers, cfg.num_experts_per_tok
    assert rec.shape == (4, 14, L, K) and rec.dtype == torch.int16
    m = data.batch["attention_mask"].bool()
    assert bool((rec[~m] == 0).all()) and int(rec.max()) < cfg.num_experts
    # every valid token's record lists K distinct experts
    valid = rec[m].long()
    assert bool((valid.sort(-1).values.diff(dim=-1) > 0).all())

    # the update sees the replayed ids in every layer, in the forward and in the recomputed backward
    seen = []
    mlp0 = eng.model.layers[0].mlp
    orig = type(mlp0)._forward

    def spy(self, x, x_router):
        if self is mlp0:
            seen.append(None if self.replay_routing is None else self.replay_routing.clone())
        return orig(self, x, x_router)

    type(mlp0)._forward = spy
    try:
        data.batch["old_log_probs"] = lp
        data.batch["routed_experts"] = rec
        with eng.train_mode():
            out = actor.update_policy(data)
    finally:
        type(mlp0)._forward = orig
    assert out["actor/grad_norm"][0] > 0 and len(seen) >= 4 and all(s is not None for s in seen)
    first = seen[0]
    want = rec[:2][m[:2]][:, 0].long()
    assert torch.equal(first, want)
    assert all(layer.mlp.replay_routing is None for layer in eng.model.layers)  # cleared after the backward

    # after the step the router has moved: free routing differs from the record somewhere, replayed log-probs follow
    # the record
    with eng.eval_mode():
        actor.router_replay = "disabled"
        free, _ = actor.compute_log_prob(data.select(batch_keys=["responses", "input_ids", "attention_mask", "position_ids"]))
        now = torch.stack([l.mlp.last_routing for l in eng.model.layers], 1)
        actor.router_replay = "R3"  # replay a given record in compute_log_prob
        replayed, _ = actor.compute_log_prob(data)
    assert replayed.shape == free.shape and torch.isfinite(replayed).all()
    if not torch.equal(now.sort(-1).values, rec[2:][m[2:]].long().sort(-1).values):
        assert not torch.allclose(free, replayed)


def test_replay_of_the_own_record_changes_nothing():
    cfg, eng, actor = _actor("R2")
    data = _batch(cfg, seed=1)
    with eng.eval_mode():
        lp, _ = actor.compute_log_prob(data)
        data.batch["routed_experts"] = actor.last_routed_experts
        actor.router_replay = "R3"
        lp2, _ = actor.compute_log_prob(data)
    torch.testing.assert_close(lp, lp2, atol=1e-6, rtol=1e-6)


def test_dense_models_and_missing_records_are_refused():
    import pytest

    eng = NativeEngine(preset("tiny-qwen2"), C(), C(lr=1e-3), device="cpu", seed=1).initialize()
    with pytest.raises(ValueError, match="mixture-of-experts"):
        DataParallelPPOActor(FSDPActorConfig(ppo_mini_batch_size=2, router_replay={"mode": "R2"}), eng)
    cfg, eng2, actor = _actor("R2")
    data = _batch(cfg)
    data.batch["old_log_probs"] = torch.zeros(4, 8)
    with pytest.raises(AssertionError, match="routed_experts"), eng2.train_mode():
        actor.update_policy(data)


def test_grpo_with_r2_replay_end_to_end(tmp_path, monkeypatch):
    """The trainer path: compute_log_prob's record travels with the batch into update_actor (two workers, two
    mini-batches per step so that the second one trains after the router has moved)."""
    import json
    import math

    from test_e2e_grpo_on_cpu import _overrides

    from verl_b200.trainer.main_ppo import run_ppo
    from verl_b200.utils.config import compose

    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    extra = ["actor_rollout_ref.model.path=preset:tiny-qwen3-moe", "actor_rollout_ref.actor.router_replay.mode=R2",
             "trainer.experiment_name=r2", "trainer.save_freq=-1", "data.max_response_length=16",
             "actor_rollout_ref.actor.ppo_mini_batch_size=4", "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=4"]
    trainer = run_ppo(compose("ppo_trainer", _overrides(tmp_path, extra)), spmd=False)
    assert trainer.global_steps == 2 and "routed_experts" in trainer._last_batch.batch.keys()
    m = [json.loads(l) for l in open(tmp_path / "logs" / "cpu_e2e" / "r2.jsonl")][-1]["data"]
    for key in ("actor/pg_loss", "actor/grad_norm", "actor/ppo_kl"):
        assert key in m and math.isfinite(m[key]), key


def test_rollout_records_the_routing_of_every_input_token():
    """R3 producer: chunked prefill + burst decode record, per request, the experts of every input token; they equal the
    routing of one full forward over the finished sequence."""
    from verl_b200.models import CausalLM, PackedBatch
    from verl_b200.rollout import NativeRolloutEngine, SamplingParams
    from verl_b200.rollout.postprocess import assemble_rollout_batch

    cfg = preset("tiny-qwen3-moe")
    model = CausalLM(cfg, dtype=torch.float32).init_weights(7)
    eng = NativeRolloutEngine(model, max_num_seqs=4, max_model_len=64, max_num_batched_tokens=8, num_blocks=32, decode_burst=4,
                              record_routing=True)
    assert not eng.enable_prefix_caching
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, 1900, (n,), generator=g).tolist() for n in (13, 5, 9)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=7, ignore_eos=True))
    L, K = cfg.num_hidden_layers, cfg.num_experts_per_tok
    for p, o in zip(prompts, outs):
        seq = torch.tensor(p + list(o.token_ids))
        assert o.routed_experts.shape == (len(seq), L, K)
        with torch.no_grad():
            model(PackedBatch(seq, torch.arange(len(seq)), torch.tensor([0, len(seq)], dtype=torch.int32), len(seq)))
        full = torch.stack([l.mlp.last_routing for l in model.layers], 1)
        got = torch.from_numpy(o.routed_experts).long()
        # every token but the last one was an input of the engine
        assert torch.equal(got[:-1].sort(-1).values, full[:-1].sort(-1).values)
        assert bool((got[-1] == 0).all())
    # the padded batch carries them aligned with input_ids
    P = 16
    ids = torch.zeros(3, P, dtype=torch.long)
    mask = torch.zeros(3, P, dtype=torch.long)
    for i, p in enumerate(prompts):
        ids[i, P - len(p):] = torch.tensor(p)
        mask[i, P - len(p):] = 1
    batch = assemble_rollout_batch(ids, mask, outs, 8, pad_token_id=0)
    re = batch.batch["routed_experts"]
    assert re.shape == (3, P + 8, L, K) and re.dtype == torch.int16
    assert torch.equal(re[1, P - 5 : P + 7], torch.from_numpy(outs[1].routed_experts)) and bool((re[1, : P - 5] == 0).all())


import pytest


@pytest.mark.parametrize("agent", [False, True, "tool"])
def test_grpo_with_r3_replay_end_to_end(tmp_path, monkeypatch, agent):
    """R3: the rollout's record is replayed in compute_log_prob and in the update (batch generation, and the server
    path of the single-turn agent loop, where the record travels with the HTTP response)."""
    import json
    import math

    from test_e2e_grpo_on_cpu import _overrides

    from verl_b200.trainer.main_ppo import run_ppo
    from verl_b200.utils.config import compose

    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    extra = ["actor_rollout_ref.model.path=preset:tiny-qwen3-moe", "actor_rollout_ref.actor.router_replay.mode=R3",
             "actor_rollout_ref.rollout.enable_rollout_routing_replay=true", "trainer.experiment_name=r3", "trainer.save_freq=-1",
             "data.max_response_length=16", "trainer.n_gpus_per_node=1"]
    if agent:
        extra += ["actor_rollout_ref.rollout.agent.use_agent_loop=true", "actor_rollout_ref.rollout.agent.num_workers=2",
                  "data.return_raw_chat=true"]
    if agent == "tool":  # the tool-calling state machine: the latest generation call's record is the sequence's record
        extra += ["actor_rollout_ref.rollout.multi_turn.enable=true", "actor_rollout_ref.rollout.multi_turn.max_assistant_turns=2",
                  "actor_rollout_ref.rollout.agent.default_agent_loop=tool_agent"]
    trainer = run_ppo(compose("ppo_trainer", _overrides(tmp_path, extra)), spmd=True)
    assert trainer.global_steps == 2 and "routed_experts" in trainer._last_batch.batch.keys()
    m = [json.loads(l) for l in open(tmp_path / "logs" / "cpu_e2e" / "r3.jsonl")][-1]["data"]
    for key in ("actor/pg_loss", "actor/grad_norm", "training/rollout_probs_diff_mean"):
        assert key in m and math.isfinite(m[key]), key
    # same weights and the same experts in the rollout and in the trainer's log-prob pass
    assert m["training/rollout_probs_diff_mean"] < 1e-3
