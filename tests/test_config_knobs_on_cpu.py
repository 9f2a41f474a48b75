"""Config fields that the reference's users set: each one changes what it names (or is refused), none is silently dropped."""
import os
import sys

import pytest
import torch

from verl_b200 import DataProto
from verl_b200.models import preset
from verl_b200.workers.actor.dp_actor import DataParallelPPOActor
from verl_b200.workers.config import FSDPActorConfig
from verl_b200.workers.engine.native import NativeEngine


class C(dict):
    __getattr__ = dict.get


def _data(B=8, P=4, R=6, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(3, 2000, (B, P + R), generator=g)
    mask = torch.ones(B, P + R, dtype=torch.long)
    pos = (mask.cumsum(-1) - 1).clamp(min=0)
    return DataProto.from_dict({"input_ids": ids, "attention_mask": mask, "position_ids": pos, "responses": ids[:, P:],
                                "response_mask": mask[:, P:], "advantages": torch.randn(B, R, generator=g),
                                "old_log_probs": -torch.rand(B, R, generator=g)}, meta_info={"temperature": 1.0})


def test_actor_shuffle_changes_the_mini_batches_reproducibly():
    seen = []

    def run(shuffle, seed):
        eng = NativeEngine(preset("tiny-qwen2"), C(), C(lr=1e-3), device="cpu", seed=1).initialize()
        actor = DataParallelPPOActor(FSDPActorConfig(ppo_mini_batch_size=4, ppo_micro_batch_size_per_gpu=4, ppo_epochs=2,
                                                     use_kl_loss=False, shuffle=shuffle, data_loader_seed=seed), eng)
        order = []
        orig = actor._forward_micro_batch
        actor._forward_micro_batch = lambda mb, *a, **k: (order.append(mb.batch["input_ids"][:, 0].tolist()), orig(mb, *a, **k))[1]
        with eng.train_mode():
            actor.update_policy(_data())
        return order

    plain, a, a2, b = run(False, 1), run(True, 1), run(True, 1), run(True, 2)
    first = _data().batch["input_ids"][:, 0].tolist()
    assert plain == [first[:4], first[4:], first[:4], first[4:]]
    assert a == a2 and a != plain and a != b and a[:2] != a[2:]           # reproducible, seeded, a new order every epoch
    assert sorted(sum(a[:2], [])) == sorted(first)                         # every sample once per epoch


def test_role_grad_clip_replaces_the_engine_default_only_when_it_alone_was_changed():
    from verl_b200.workers.engine_workers import _role_clip

    assert _role_clip(C(grad_clip=1.0, optim=C(clip_grad=1.0))) is None
    assert _role_clip(C(grad_clip=0.3, optim=C(clip_grad=1.0))) == 0.3
    assert _role_clip(C(grad_clip=0.3, optim=C(clip_grad=0.5))) is None
    norms = {}
    for clip in (None, 1e-3):
        eng = NativeEngine(preset("tiny-qwen2"), C(), C(lr=1.0, clip_grad=1.0, weight_decay=0.0), device="cpu", seed=1).initialize()
        eng.clip_grad_override = clip
        actor = DataParallelPPOActor(FSDPActorConfig(ppo_mini_batch_size=8, ppo_micro_batch_size_per_gpu=8, use_kl_loss=False), eng)
        before = {k: v.clone() for k, v in eng.zero.named_full_tensors()}
        with eng.train_mode():
            actor.update_policy(_data())
        norms[clip] = sum(float((v.float() - before[k].float()).abs().sum()) for k, v in eng.zero.named_full_tensors())
    assert norms[None] > 0 and norms[1e-3] > 0


def test_full_determinism_switch_of_the_engine():
    try:
        NativeEngine(preset("tiny-qwen2"), C(full_determinism=True), C(lr=1e-3), device="cpu", seed=5)
        assert torch.are_deterministic_algorithms_enabled() and os.environ["PYTHONHASHSEED"] == "5"
    finally:
        torch.use_deterministic_algorithms(False)


def test_custom_agent_loops_from_a_config_file(tmp_path):
    import asyncio

    from verl_b200.experimental.agent_loop.agent_loop import AgentLoopWorker, _agent_loop_registry

    (tmp_path / "my_loops.py").write_text(
        "from verl_b200.experimental.agent_loop.agent_loop import AgentLoopBase, AgentLoopOutput, AgentLoopMetrics\n"
        "class EchoLoop(AgentLoopBase):\n"
        "    def __init__(self, suffix=0, **kw):\n"
        "        super().__init__(**kw)\n"
        "        self.suffix = suffix\n"
        "    async def run(self, sampling_params, **kwargs):\n"
        "        p = [int(t) for t in kwargs['raw_prompt']]\n"
        "        return AgentLoopOutput(prompt_ids=p, response_ids=p[::-1] + [self.suffix], response_mask=[1] * (len(p) + 1),\n"
        "                               response_logprobs=[0.0] * (len(p) + 1), num_turns=2, metrics=AgentLoopMetrics())\n")
    (tmp_path / "loops.yaml").write_text("- name: echo\n  _target_: my_loops.EchoLoop\n  suffix: 7\n")
    sys.path.insert(0, str(tmp_path))
    try:
        from verl_b200.utils.config import compose
        from verl_b200.utils.tokenizer import IntTokenizer

        cfg = compose("ppo_trainer", ["actor_rollout_ref.model.path=preset:tiny-qwen2", "data.max_prompt_length=8",
                                      "data.max_response_length=8", f"actor_rollout_ref.rollout.agent.agent_loop_config_path={tmp_path}/loops.yaml",
                                      "actor_rollout_ref.model.custom_chat_template=TEMPLATE"])
        tok = IntTokenizer(2048)
        w = AgentLoopWorker(cfg, [], tok)
        assert tok.chat_template == "TEMPLATE" and "echo" in _agent_loop_registry
        import numpy as np

        raw = np.empty(2, dtype=object)
        raw[:] = [[5, 6, 7], [9, 8]]
        names = np.array(["echo", "echo"], dtype=object)
        out = asyncio.run(w.generate_sequences(DataProto.from_dict(tensors={"dummy": torch.zeros(2, 1)},
                                                                   non_tensors={"raw_prompt": raw, "agent_name": names})))
        assert out.batch["responses"][0, :4].tolist() == [7, 6, 5, 7] and out.batch["responses"][1, :3].tolist() == [8, 9, 7]
    finally:
        sys.path.remove(str(tmp_path))
        _agent_loop_registry.pop("echo", None)
        sys.modules.pop("my_loops", None)


def test_frozen_vision_tower_stays_bit_identical_while_the_decoder_trains():
    from verl_b200.models.vision import get_rope_index
    import numpy as np

    cfg = preset("tiny-qwen2-vl")
    eng = NativeEngine(cfg, C(), C(lr=1e-2, clip_grad=1.0, weight_decay=0.1), device="cpu", seed=3,
                       frozen_prefixes=("visual.",)).initialize()
    actor = DataParallelPPOActor(FSDPActorConfig(ppo_mini_batch_size=2, ppo_micro_batch_size_per_gpu=1, use_kl_loss=False), eng)
    g = torch.Generator().manual_seed(2)
    P, R, B, tok = 12, 6, 2, cfg.image_token_id
    grid = torch.tensor([[1, 4, 4]])
    ids = torch.zeros(B, P + R, dtype=torch.long)
    mask = torch.zeros(B, P + R, dtype=torch.long)
    pos = torch.zeros(B, 4, P + R, dtype=torch.long)
    mm = []
    for i in range(B):
        seq = torch.tensor([5 + i, 2002] + [tok] * 4 + [9, 11, 13] + torch.randint(3, 1900, (R,), generator=g).tolist())
        lo = P - 9
        ids[i, lo : lo + len(seq)], mask[i, lo : lo + len(seq)] = seq, 1
        pos[i, 1:, lo : lo + len(seq)] = get_rope_index(seq, grid, tok, 2)[0]
        pos[i, 0, lo : lo + len(seq)] = torch.arange(len(seq))
        mm.append({"pixel_values": torch.randn(16, 96, generator=g), "image_grid_thw": grid})
    data = DataProto.from_dict({"input_ids": ids, "attention_mask": mask, "position_ids": pos, "responses": ids[:, P:],
                                "response_mask": mask[:, P:], "old_log_probs": -torch.rand(B, R, generator=g),
                                "advantages": torch.randn(B, R, generator=g)},
                               non_tensors={"multi_modal_inputs": np.array(mm, dtype=object)}, meta_info={"temperature": 1.0})
    before = {k: v.clone() for k, v in eng.zero.named_full_tensors()}
    with eng.train_mode():
        for _ in range(2):
            out = actor.update_policy(data)
    assert out["actor/grad_norm"][0] > 0
    after = dict(eng.zero.named_full_tensors())
    vis = [k for k in before if k.startswith("visual.")]
    assert vis and all(torch.equal(before[k], after[k]) for k in vis)
    assert not torch.equal(before["layers.0.self_attn.qkv_proj.weight"], after["layers.0.self_attn.qkv_proj.weight"])
    with pytest.raises(ValueError, match="no parameter name starts with"):
        NativeEngine(preset("tiny-qwen2"), C(), C(lr=1e-3), device="cpu", seed=1, frozen_prefixes=("visual.",)).initialize()


def test_checkpoint_engine_from_its_config_section():
    from verl_b200.checkpoint_engine import build_checkpoint_engine
    from verl_b200.workers.config import CheckpointEngineConfig

    e = build_checkpoint_engine(CheckpointEngineConfig(backend="nccl", update_weights_bucket_megabytes=3,
                                                       engine_kwargs={"nccl": {"src": 1}}), is_master=False)
    assert type(e).__name__ == "NCCLCheckpointEngine" and e.bucket_size == 3 << 20 and e.src == 1
    assert build_checkpoint_engine({"backend": "naive"}).bucket_size == 2048 << 20
    with pytest.raises(ValueError, match="Unknown checkpoint engine backend"):
        build_checkpoint_engine({"backend": "nixl2"})


def test_megatron_strategy_command_lines_map_onto_the_native_engine(capsys):
    from verl_b200.utils.config import compose, translate_megatron_overrides

    ov = ["actor_rollout_ref.actor.strategy=megatron", "actor_rollout_ref.actor.megatron.tensor_model_parallel_size=2",
          "actor_rollout_ref.actor.megatron.pipeline_model_parallel_size=2", "actor_rollout_ref.actor.megatron.param_offload=true",
          "actor_rollout_ref.ref.megatron.tensor_model_parallel_size=2", "critic.strategy=megatron",
          "critic.megatron.expert_model_parallel_size=4", "actor_rollout_ref.actor.megatron.use_mbridge=true",
          "+actor_rollout_ref.actor.megatron.override_transformer_config.recompute_granularity=full",
          "actor_rollout_ref.actor.optim.lr_decay_style=cosine", "actor_rollout_ref.actor.optim.lr=2e-6",
          "actor_rollout_ref.model.path=preset:tiny-qwen2"]
    out, dropped = translate_megatron_overrides(ov)
    assert "actor_rollout_ref.actor.fsdp_config.tensor_model_parallel_size=2" in out and "critic.model.fsdp_config.expert_model_parallel_size=4" in out
    assert len(dropped) == 2 and all("megatron" not in o for o in out)
    cfg = compose("ppo_megatron_trainer", ov)
    a = cfg.actor_rollout_ref.actor
    assert a.strategy == "fsdp" and a.fsdp_config.tensor_model_parallel_size == 2 and a.fsdp_config.pipeline_model_parallel_size == 2
    assert a.fsdp_config.param_offload is True and a.optim.lr_scheduler_type == "cosine" and a.optim.lr == 2e-6
    assert cfg.actor_rollout_ref.ref.fsdp_config.tensor_model_parallel_size == 2
    assert cfg.critic.strategy == "fsdp" and cfg.critic.model.fsdp_config.expert_model_parallel_size == 4
    assert "left out" in capsys.readouterr().out
    with pytest.raises(NotImplementedError, match="virtual pipeline"):
        translate_megatron_overrides(["actor_rollout_ref.actor.megatron.virtual_pipeline_model_parallel_size=2"])
    with pytest.raises(NotImplementedError, match="lr_decay_style"):
        translate_megatron_overrides(["actor_rollout_ref.actor.optim.lr_decay_style=inverse-square-root"])


def test_megatron_style_command_line_trains_with_tensor_parallelism(tmp_path, monkeypatch):
    """The reference's Megatron launch flags, end to end: two gloo workers, the actor sharded over a tensor-parallel
    group of two as ``actor.megatron.tensor_model_parallel_size=2`` asks."""
    import json
    import math

    from test_e2e_grpo_on_cpu import _overrides

    from verl_b200.trainer.main_ppo import run_ppo
    from verl_b200.utils.config import compose

    monkeypatch.setenv("VERL_FILE_LOGGER_ROOT", str(tmp_path / "logs"))
    extra = ["actor_rollout_ref.actor.strategy=megatron", "actor_rollout_ref.actor.megatron.tensor_model_parallel_size=2",
             "actor_rollout_ref.ref.strategy=megatron", "actor_rollout_ref.ref.megatron.tensor_model_parallel_size=2",
             "actor_rollout_ref.actor.megatron.use_distributed_optimizer=true", "trainer.experiment_name=mcore",
             "trainer.save_freq=-1", "trainer.total_training_steps=1", "data.max_response_length=16"]
    trainer = run_ppo(compose("ppo_megatron_trainer", _overrides(tmp_path, extra)), spmd=False)
    assert trainer.global_steps == 1
    assert trainer.config.actor_rollout_ref.actor.fsdp_config.tensor_model_parallel_size == 2
    m = [json.loads(l) for l in open(tmp_path / "logs" / "cpu_e2e" / "mcore.jsonl")][-1]["data"]
    assert math.isfinite(m["actor/pg_loss"]) and m["actor/grad_norm"] > 0
