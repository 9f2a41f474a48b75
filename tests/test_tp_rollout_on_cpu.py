"""Tensor-parallel rollout replica on 2 gloo ranks: same tokens as the unsharded model (dense, replicated KV heads,
expert-parallel MoE), and the TP planner's slices."""

import os
import subprocess
import sys

import pytest
import torch


def test_tp2_replica_matches_single_rank():
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29350 + os.getpid() % 300), os.path.join(here, "_tp_rollout_worker.py"), "cpu"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "TP_ROLLOUT_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-5000:])


def test_tp_slices_cover_the_model_once():
    """Summing what the ranks' row-parallel slices compute, and concatenating the column-parallel ones, gives the
    whole layer; KV heads are replicated when there are fewer of them than ranks."""
    from verl_b200.models import CausalLM, preset
    from verl_b200.parallel.reshard import shard_state_dict, tp_model_config

    cfg = preset("tiny-qwen2", num_attention_heads=8, num_key_value_heads=2, hidden_size=256, intermediate_size=512)
    full = dict(CausalLM(cfg, dtype=torch.float32).init_weights(0).state_dict())
    tp = 4
    parts = [shard_state_dict(cfg, full, r, tp) for r in range(tp)]
    D = cfg.head_dim
    name = "layers.0.self_attn.qkv_proj.weight"
    q = torch.cat([p[name][: cfg.q_size // tp] for p in parts])
    assert torch.equal(q, full[name][: cfg.q_size])
    for r in range(tp):
        k = parts[r][name][cfg.q_size // tp : cfg.q_size // tp + D]
        head = r // (tp // cfg.num_key_value_heads)
        assert torch.equal(k, full[name][cfg.q_size + head * D : cfg.q_size + (head + 1) * D])
    o = torch.cat([p["layers.0.self_attn.o_proj.weight"] for p in parts], dim=1)
    assert torch.equal(o, full["layers.0.self_attn.o_proj.weight"])
    c4 = tp_model_config(cfg, 1, tp)
    assert (c4.num_attention_heads, c4.num_key_value_heads, c4.head_dim) == (2, 1, D)
    with pytest.raises(ValueError):
        tp_model_config(cfg, 0, 3)
