"""Small modules that carry the reference's helper APIs: micro-batch preparation over TensorDicts, the checkpoint
handler, vocabulary-parallel log-probs, base interfaces, the redirect table of the ``verl`` alias package."""
import os
import subprocess
import sys

import pytest
import torch


def _jagged(rows):
    return torch.nested.as_nested_tensor(rows, layout=torch.jagged)


def test_prepare_micro_batches_and_postprocess_round_trip():
    from verl_b200.utils import tensordict_utils as tu
    from verl_b200.workers.engine.utils import postprocess_batch_func, prepare_micro_batches

    lens = [5, 3, 9, 2, 7, 4, 8, 1]
    rows = [torch.arange(n) + 100 * i for i, n in enumerate(lens)]
    data = tu.get_tensordict({"input_ids": _jagged(rows)}, {"use_dynamic_bsz": True, "max_token_len_per_gpu": 12})
    mbs, idx = prepare_micro_batches(data)
    assert sorted(i for p in idx for i in p) == list(range(len(lens))) and len(mbs) >= 4
    for mb, p in zip(mbs, idx):
        assert sum(lens[i] for i in p) <= 12 and [r.tolist() for r in mb["input_ids"].unbind()] == [rows[i].tolist() for i in p]
    outs = [{"model_output": {"log_probs": _jagged([r.float() * 2 for r in mb["input_ids"].unbind()])},
             "loss": float(k), "metrics": {"m": k}} for k, mb in enumerate(mbs)]
    res = postprocess_batch_func(outs, idx, data)
    got = [r.tolist() for r in res["model_output"]["log_probs"].unbind()]
    assert got == [(r.float() * 2).tolist() for r in rows]  # original row order restored
    assert res["loss"] == [float(k) for k in range(len(mbs))] and res["metrics"]["m"] == list(range(len(mbs)))

    # the sequence-parallel size multiplies the budget; fixed-size chunks when dynamic batching is off
    data2 = tu.get_tensordict({"input_ids": _jagged(rows)}, {"use_dynamic_bsz": True, "max_token_len_per_gpu": 12, "sp_size": 2})
    assert len(prepare_micro_batches(data2)[0]) < len(mbs)
    data3 = tu.get_tensordict({"input_ids": _jagged(rows)}, {"use_dynamic_bsz": False, "micro_batch_size_per_gpu": 2})
    mbs3, idx3 = prepare_micro_batches(data3)
    assert idx3 is None and [len(m) for m in mbs3] == [2, 2, 2, 2]
    res3 = postprocess_batch_func([{"model_output": {"x": m["input_ids"]}, "loss": 0.0} for m in mbs3], None, data3)
    assert [r.tolist() for r in res3["model_output"]["x"].unbind()] == [r.tolist() for r in rows]


def test_enable_full_determinism_seeds_everything():
    import random

    import numpy as np

    from verl_b200.workers.engine.utils import enable_full_determinism

    try:
        enable_full_determinism(7)
        a = (random.random(), float(np.random.rand()), float(torch.rand(1)))
        enable_full_determinism(7)
        assert a == (random.random(), float(np.random.rand()), float(torch.rand(1)))
        assert torch.are_deterministic_algorithms_enabled()
    finally:
        torch.use_deterministic_algorithms(False)


class _Engine:
    def __init__(self):
        self.state, self.saved, self.loaded = {"w": 0}, [], None

    def is_mp_src_rank_with_outputs(self):
        return True

    def get_data_parallel_rank(self):
        return 0

    def save_checkpoint(self, local_path, global_step=0, max_ckpt_to_keep=None, **kw):
        os.makedirs(local_path, exist_ok=True)
        torch.save(dict(self.state), os.path.join(local_path, "model.pt"))
        self.saved.append(global_step)

    def load_checkpoint(self, local_path, **kw):
        self.state, self.loaded = torch.load(os.path.join(local_path, "model.pt")), local_path


class _Loader:
    def __init__(self):
        self.pos = 0

    def state_dict(self):
        return {"pos": self.pos}

    def load_state_dict(self, sd):
        self.pos = sd["pos"]


def test_checkpoint_handler_saves_rotates_and_resumes(tmp_path):
    from verl_b200.utils.checkpoint.checkpoint_handler import CheckpointHandler, extract_step
    from verl_b200.utils.checkpoint.checkpoint_manager import get_checkpoint_tracker_filename

    root = str(tmp_path / "ckpt")
    eng, loader = _Engine(), _Loader()
    h = CheckpointHandler(eng, loader, default_local_dir=root, max_ckpt_to_keep=2)
    assert h.load_checkpoint() == 0  # nothing to resume from
    for step in (2, 4, 6):
        eng.state["w"], loader.pos = step * 10, step
        h.save_checkpoint(step)
    assert sorted(os.listdir(root)) == sorted(["global_step_4", "global_step_6", os.path.basename(get_checkpoint_tracker_filename(root))])
    assert open(get_checkpoint_tracker_filename(root)).read().strip() == "6"

    eng2, loader2 = _Engine(), _Loader()
    h2 = CheckpointHandler(eng2, loader2, default_local_dir=root)
    assert h2.load_checkpoint() == 6 and eng2.state["w"] == 60 and loader2.pos == 6
    h3 = CheckpointHandler(_Engine(), _Loader(), default_local_dir=root, resume_mode="resume_path",
                           resume_from_path=os.path.join(root, "global_step_4"))
    assert h3.load_checkpoint() == 4 and h3.engine.state["w"] == 40
    assert CheckpointHandler(_Engine(), _Loader(), default_local_dir=root, resume_mode="disable").load_checkpoint() == 0
    with pytest.raises(ValueError):
        CheckpointHandler(_Engine(), _Loader(), default_local_dir=root, resume_mode="bogus").load_checkpoint()
    assert extract_step("/a/global_step_12/actor") == 12 and extract_step("/a/b") is None


def test_vocab_parallel_single_rank_matches_dense():
    from verl_b200.parallel.vocab_parallel import pad_to_sequence_parallel, vocab_parallel_entropy, vocab_parallel_log_probs_from_logits

    x = torch.randn(4, 11, dtype=torch.float64, requires_grad=True)
    y = torch.randint(0, 11, (4,))
    assert torch.autograd.gradcheck(lambda t: vocab_parallel_log_probs_from_logits(t.float(), y).double(), (x,), atol=1e-3, eps=1e-3)
    ls = torch.log_softmax(x.float(), -1)
    torch.testing.assert_close(vocab_parallel_entropy(x.float()), -(ls.exp() * ls).sum(-1))
    assert pad_to_sequence_parallel(torch.ones(7, 3), 4).shape == (8, 3) and pad_to_sequence_parallel(torch.ones(8), 4).shape == (8,)


def test_vocab_parallel_two_ranks_match_dense():
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29950 + os.getpid() % 40), os.path.join(here, "_vocab_parallel_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "VOCAB_PARALLEL_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])


def test_base_interfaces_and_redirected_paths():
    from verl.models.transformers.tiled_mlp import TiledMLP  # noqa: F401
    from verl.utils.checkpoint.checkpoint_handler import CheckpointHandler  # noqa: F401
    from verl.utils.experimental.torch_functional import FusedLinearForPPO
    from verl.utils.megatron.tensor_parallel import vocab_parallel_entropy  # noqa: F401
    from verl.utils.metric.utils import Metric, reduce_metrics  # noqa: F401
    from verl.utils.transformers_compat import is_transformers_version_in_range
    from verl.workers.actor.base import BasePPOActor
    from verl.workers.critic.base import BasePPOCritic
    from verl.workers.engine.fsdp.utils import prepare_micro_batches  # noqa: F401
    from verl.workers.megatron_workers import ActorRolloutRefWorker
    from verl.workers.reward_model.base import BasePPORewardModel
    from verl.workers.rollout.vllm_rollout.vllm_rollout import ServerAdapter

    import verl_b200.workers.engine_workers as ew
    from verl_b200.workers.rollout.native_rollout import ServerAdapter as Native

    assert ActorRolloutRefWorker is ew.ActorRolloutRefWorker and ServerAdapter is Native
    for base in (BasePPOActor, BasePPOCritic, BasePPORewardModel):
        with pytest.raises(TypeError):
            base(config=None)  # abstract
    assert is_transformers_version_in_range(min_version="4.0") and not is_transformers_version_in_range(max_version="1.0")
    h, w, ids = torch.randn(6, 8), torch.randn(13, 8), torch.randint(0, 13, (6,))
    lp, ent = FusedLinearForPPO()(h, w, ids)
    ls = torch.log_softmax(h @ w.T, -1)
    torch.testing.assert_close(lp, ls.gather(-1, ids[:, None])[:, 0]) and torch.testing.assert_close(ent, -(ls.exp() * ls).sum(-1))


def test_checkpoint_manager_contents_retention_and_rng(tmp_path):
    import random

    import numpy as np

    from verl_b200.models import preset
    from verl_b200.utils.checkpoint.checkpoint_manager import BaseCheckpointManager, NativeCheckpointManager
    from verl_b200.workers.engine.native import NativeEngine

    class C(dict):
        __getattr__ = dict.get

    m = BaseCheckpointManager(model=None, checkpoint_config={"save_contents": ["model", "hf_model"], "load_contents": ["model"]})
    assert m.should_save_model and m.should_save_hf_model and not m.should_save_optimizer and not m.should_save_extra
    assert m.should_load_model and not m.should_load_optimizer
    with pytest.raises(NotImplementedError):
        m.save_checkpoint("x")
    assert BaseCheckpointManager.checkpath("a", None) == (True, "a") and BaseCheckpointManager.checkpath(None, "h") == (False, "h")
    st = BaseCheckpointManager.get_rng_state()
    a = (random.random(), float(np.random.rand()), float(torch.rand(1)))
    BaseCheckpointManager.load_rng_state(st)
    assert a == (random.random(), float(np.random.rand()), float(torch.rand(1)))

    # the engine's own saves: at most two folders stay, the weights of the newest come back
    eng = NativeEngine(preset("tiny-qwen2"), C(), C(lr=1e-3), device="cpu", seed=1).initialize()
    for step in (1, 2, 3):
        eng.save_checkpoint(str(tmp_path / f"global_step_{step}"), global_step=step, max_ckpt_to_keep=2)
    assert sorted(os.listdir(tmp_path)) == ["global_step_2", "global_step_3"]
    eng2 = NativeEngine(preset("tiny-qwen2"), C(), C(lr=1e-3), device="cpu", seed=9).initialize()
    mgr = NativeCheckpointManager(eng2, checkpoint_config={"load_contents": ["model"]})
    mgr.load_checkpoint(str(tmp_path / "global_step_3"))
    for (k, a_), (_, b_) in zip(eng.zero.named_full_tensors(), eng2.zero.named_full_tensors()):
        assert torch.equal(a_, b_), k


def test_dataset_split_metric_chain_profiler_predicates_and_worker_dispatch_info(tmp_path):
    import json

    from verl_b200.single_controller.base import Worker
    from verl_b200.utils.dataset.rl_dataset import RLHFDataset, get_dataset_class
    from verl_b200.utils.metric import AggregationType, Metric
    from verl_b200.utils.profiler.profile import DistProfiler, mark_annotate
    from verl_b200.utils.tokenizer import IntTokenizer

    f = tmp_path / "p.jsonl"
    f.write_text("\n".join(json.dumps({"prompt": " ".join(str(3 + j) for j in range(2 + i)), "data_source": "x"}) for i in range(7)))
    ds = RLHFDataset(str(f), IntTokenizer(64), {"max_prompt_length": 6, "filter_overlong_prompts": False})
    parts = ds.split(3)
    assert [len(p) for p in parts] == [3, 2, 2] and parts[1][0]["raw_prompt_ids"] == ds[3]["raw_prompt_ids"]
    with pytest.raises(ValueError):
        ds.split(0)
    ds.filter_overlong_prompts = True
    assert len(ds.maybe_filter_out_long_prompts()) == 5  # prompts of 2..6 tokens fit
    assert get_dataset_class({"custom_cls": {"path": None, "name": None}}) is RLHFDataset
    (tmp_path / "mine.py").write_text("class D:\n    def __len__(self):\n        return 0\n    def __getitem__(self, i):\n        raise IndexError\nX = 3\n")
    assert get_dataset_class({"custom_cls": {"path": str(tmp_path / "mine.py"), "name": "D"}}).__name__ == "D"
    with pytest.raises(TypeError):
        get_dataset_class({"custom_cls": {"path": str(tmp_path / "mine.py"), "name": "X"}})

    m = Metric.chain([Metric("max", [1, 5]), Metric("max", 3)])
    assert m.aggregation == AggregationType.MAX and m.aggregate() == 5.0 and Metric.chain([]).aggregation == AggregationType.MEAN

    p = DistProfiler(1, {"enable": True, "ranks": [1], "tool": "none"})
    assert p.check_enable() and p.check_this_rank() and not p.check_this_step() and not p.is_discrete_mode()
    p.start()
    assert p.check_this_step()
    p.stop()
    assert not p.check_this_step() and not DistProfiler(0, {"enable": True, "ranks": [1]}).check_this_rank()
    assert mark_annotate("phase")(lambda a, b=1: a + b)(2, b=3) == 5

    w = Worker()
    w._register_dispatch_collect_info("actor", 3, True)
    assert w.get_dispatch_collect() == {"dispatch_dp_rank": {"actor": 3}, "collect_dp_rank": {"actor": True}}
    w.set_dispatch_collect("ref", {"actor": 3}, {"actor": True})
    assert w._query_dispatch_info("ref") == 3 and w.query_collect_info("ref")
