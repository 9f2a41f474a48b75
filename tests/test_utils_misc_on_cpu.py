"""Small utilities: rollout skip / trace, memory buffers, prefix grouper, fs and import helpers."""

import asyncio
import json
import os

import numpy as np
import torch


def test_prefix_grouper_roundtrip_and_mask():
    from verl_b200.trainer.ppo import prefix_grouper_utils as pg

    P, R = 6, 5
    prompts = torch.tensor([[0, 0, 5, 6, 7, 8]] * 3 + [[0, 9, 9, 9, 9, 9]] * 2)
    responses = torch.tensor([[1, 2, 3, 0, 0], [4, 5, 0, 0, 0], [6, 7, 8, 9, 1], [2, 2, 0, 0, 0], [3, 0, 0, 0, 0]])
    mask = torch.cat([(prompts != 0).long(), (responses != 0).long()], 1)
    groups = pg.build_prefix_groups(prompts, responses, mask)
    assert [g.rows for g in groups] == [[0, 1, 2], [3, 4]]
    ids, pos, cu, seg, where = pg.pack_with_shared_prefix(groups)
    assert cu.tolist() == [0, 4 + 3 + 2 + 5, 14 + 5 + 2 + 1]
    assert pos[4:7].tolist() == [4, 5, 6] and pos[7:9].tolist() == [4, 5]  # every response continues after the prompt
    m = pg.prefix_sharing_mask(seg, cu)
    q = where[1][0]  # first token of response 1 of group 0
    assert m[q, :4].all() and not m[q, 4:7].any() and m[q, q]
    vals = torch.arange(ids.numel(), dtype=torch.float32)
    out = pg.unpack_shared_prefix(vals, where, 5, R)
    assert out[0, 1] == where[0][0] and out[2, 4] == where[2][0] + 3
    assert 0.2 < pg.prefix_saving(groups) < 0.6


def test_memory_buffer_wrapper():
    from verl_b200.utils.memory_buffer import MemoryBufferModuleWrapper

    m = torch.nn.Sequential(torch.nn.Linear(8, 4), torch.nn.Linear(4, 2))
    ref = {k: v.detach().clone() for k, v in m.named_parameters()}
    w = MemoryBufferModuleWrapper(m)
    buf = w.get_memory_buffers()[torch.float32]
    for k, v in m.named_parameters():
        assert torch.equal(v, ref[k])
        assert buf.data.data_ptr() <= v.data_ptr() < buf.data.data_ptr() + buf.data.numel() * 4
    buf.data.zero_()
    assert all(float(v.abs().sum()) == 0 for v in m.parameters())


def test_rollout_trace_file_backend(tmp_path):
    from verl_b200.utils.rollout_trace import RolloutTraceConfig, rollout_trace_attr, rollout_trace_op

    RolloutTraceConfig.reset()
    RolloutTraceConfig.init("p", "e", "file", path=str(tmp_path / "t.jsonl"))

    class A:
        @rollout_trace_op
        async def step(self, x, y=2):
            return {"sum": x + y}

    async def go():
        with rollout_trace_attr(sample_index=3, step=7, rollout_n=1):
            return await A().step(1, y=5)

    assert asyncio.run(go()) == {"sum": 6}
    rows = [json.loads(l) for l in open(tmp_path / "t.jsonl")]
    assert rows[0]["inputs"] == {"x": 1, "y": 5} and rows[0]["attrs"]["step"] == 7 and rows[0]["output"] == {"sum": 6}
    RolloutTraceConfig.reset()


def test_rollout_skip_replays(tmp_path):
    from verl_b200.protocol import DataProto
    from verl_b200.utils.config import to_config
    from verl_b200.utils.rollout_skip import RolloutSkip

    cfg = to_config({"actor_rollout_ref": {"rollout": {"n": 1, "skip_dump_dir": str(tmp_path)}},
                     "trainer": {"project_name": "p", "experiment_name": "e"},
                     "data": {"train_batch_size": 2, "max_prompt_length": 4, "max_response_length": 4}})
    calls = [0]

    class WG:
        def generate_sequences(self, batch, **kw):
            calls[0] += 1
            return DataProto.from_dict(tensors={"responses": torch.full((2, 4), calls[0])})

    batch = DataProto.from_dict(tensors={"input_ids": torch.zeros(2, 4, dtype=torch.long)})
    wg = WG()
    RolloutSkip(cfg, wg).wrap_generate_sequences()
    a = wg.generate_sequences(batch)
    wg2 = WG()
    RolloutSkip(cfg, wg2).wrap_generate_sequences()
    b = wg2.generate_sequences(batch)
    assert calls[0] == 1 and torch.equal(a.batch["responses"], b.batch["responses"])


def test_fs_and_import_helpers(tmp_path):
    from verl_b200.utils import fs, import_utils, net_utils

    f = tmp_path / "x.txt"
    f.write_text("hi")
    assert fs.copy_to_local(str(f)) == str(f)
    shm = fs.copy_to_local(str(f), use_shm=True)
    assert shm.startswith("/dev/shm/") and open(shm).read() == "hi"
    os.remove(shm)
    assert import_utils.is_package_available("torch") and not import_utils.is_package_available("not_a_package_xyz")
    assert net_utils.is_ipv4("127.0.0.1") and net_utils.is_ipv6("::1") and net_utils.get_free_port() > 0
    try:
        fs.copy_to_local("hdfs://nn/path")
        raise AssertionError("expected a RuntimeError")
    except RuntimeError:
        pass


def test_diagnose_report():
    from verl_b200.utils.diagnose import collect

    info = collect()
    assert info["python"] and "torch" in info and "native_library" in info and isinstance(info["env"], dict)


def test_rollout_viewer(tmp_path):
    import json

    from verl_b200.utils.rollout_viewer import main

    for step in (1, 2):
        with open(tmp_path / f"{step}.jsonl", "w") as f:
            for i in range(3):
                f.write(json.dumps({"input": f"q{i}", "output": f"answer {i} step {step}", "score": i / 2, "step": step}) + "\n")
    text = main([str(tmp_path), "--step", "2", "--min-score", "0.5", "--sort", "score_desc"])
    assert "2 rollouts" in text and text.index("answer 2 step 2") < text.index("answer 1 step 2") and "step 1" not in text
    assert "1 rollouts" in main([str(tmp_path / "1.jsonl"), "--grep", "answer 0"])


def test_kernel_breakdown_interval_arithmetic_and_classes():
    from verl_b200.utils.profiler.kernel_breakdown import _subtract, _union, classify

    assert _union([(0, 2), (1, 3), (5, 6)]) == [[0, 3], [5, 6]]
    # communication [0,4] and [10,12]; compute covers [1,2] and [3,11]: exposed = [0,1] + [2,3] + [11,12]
    assert _subtract(_union([(0, 4), (10, 12)]), _union([(1, 2), (3, 11)])) == 3
    assert classify("void vb::gemm_kernel<256, false, false, 0>(vb::GemmParams)") == "gemm"
    assert classify("vb::flash_bwd_dq_kernel") == "attention_bwd"
    assert classify("void vb::peer_reduce_scatter_add_kernel<8, 2>") == "comm"
    assert classify("vb::adamw_kernel") == "optimizer"
    assert classify("at::native::vectorized_elementwise_kernel") == "other_torch"


def test_communicator_found_by_name_between_unrelated_processes(tmp_path):
    """Three processes with nothing in common but a group name and a registry directory build a process group; the
    late starters find the endpoint that rank 0 published."""
    import subprocess
    import sys
    import time

    from verl_b200.utils.rendezvous import lookup_endpoint

    here = os.path.dirname(os.path.abspath(__file__))
    assert lookup_endpoint("nobody", str(tmp_path), max_retries=2, interval_s=0.01) is None
    procs = []
    for rank in (2, 1, 0):  # rank 0 last: the others poll until it has published
        procs.append(subprocess.Popen([sys.executable, os.path.join(here, "_rendezvous_worker.py"), str(rank), "3", "sync-group",
                                       str(tmp_path)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
        time.sleep(0.3)
    outs = [p.communicate(timeout=300) for p in procs]
    assert all(p.returncode == 0 for p in procs), [o[1][-1500:] for o in outs]
    assert sorted(o[0].strip() for o in outs) == ["RENDEZVOUS_OK 0", "RENDEZVOUS_OK 1", "RENDEZVOUS_OK 2"]
    assert not os.path.exists(tmp_path / "sync-group.json")


def test_small_helpers_with_the_reference_names(tmp_path):
    from verl_b200.protocol import deserialize_tensordict, serialize_tensordict
    from verl_b200.utils import tensordict_utils as tu
    from verl_b200.utils import torch_functional as F_
    from verl_b200.utils.fs import verify_copy
    from verl_b200.utils.import_utils import load_class_from_fqn, load_module
    from verl_b200.utils.memory_utils import MemorySnapshotSampler, reset_memory_stats

    # tensors as bytes: dense (bf16 too) and jagged entries survive the round trip
    rows = [torch.arange(n, dtype=torch.int64) for n in (3, 1, 4)]
    td = tu.get_tensordict({"a": torch.randn(3, 5).to(torch.bfloat16), "ids": torch.nested.as_nested_tensor(rows, layout=torch.jagged)})
    back = deserialize_tensordict(serialize_tensordict(td))
    assert torch.equal(back["a"], td["a"]) and [r.tolist() for r in back["ids"].unbind()] == [r.tolist() for r in rows]
    assert tuple(back.batch_size) == (3,)
    # packed and padded log-prob helpers agree with a dense log-softmax
    g = torch.Generator().manual_seed(0)
    ids, logits = torch.randint(0, 17, (3, 9), generator=g), torch.randn(3, 9, 17, generator=g)
    mask = torch.ones(3, 9, dtype=torch.long)
    mask[0, :3] = 0
    want = torch.log_softmax(logits, -1)[:, :-1].gather(-1, ids[:, 1:, None])[..., 0][:, -4:]
    torch.testing.assert_close(F_.log_probs_from_logits_response(ids, logits, 4), want)
    idx, cu, longest = F_.get_unpad_data(mask)
    assert cu.tolist() == [0, 6, 15, 24] and longest == 9
    torch.testing.assert_close(F_.log_probs_from_logits_response_rmpad(ids, mask, logits.reshape(-1, 17)[idx], 4), want)
    lin = torch.nn.Linear(3, 2)
    lin(torch.ones(1, 3)).sum().backward()
    assert abs(F_.compute_grad_norm(lin) - (6.0 + 2.0)) < 1e-6
    # files and modules
    (tmp_path / "src" / "d").mkdir(parents=True)
    (tmp_path / "src" / "d" / "f.txt").write_text("abc")
    import shutil

    shutil.copytree(tmp_path / "src", tmp_path / "dst")
    assert verify_copy(str(tmp_path / "src"), str(tmp_path / "dst"))
    (tmp_path / "dst" / "d" / "f.txt").write_text("abcd")
    assert not verify_copy(str(tmp_path / "src"), str(tmp_path / "dst"))
    (tmp_path / "m.py").write_text("VALUE = 41\n")
    assert load_module(str(tmp_path / "m.py")).VALUE == 41 and load_module("pkg://json").dumps([1]) == "[1]"
    assert load_class_from_fqn("collections.OrderedDict").__name__ == "OrderedDict"
    reset_memory_stats()
    assert MemorySnapshotSampler(str(tmp_path / "snaps")).dump_memory_snapshot().endswith("periodic_00000.pickle")
