"""Reshard planner: ZeRO flat shards -> rollout (TP) layout, checked by executing the copy table on host arrays."""
import numpy as np
import pytest
import torch

from verl_b200.models import build_model, preset
from verl_b200.parallel.reshard import build_dest_layout, execute_on_host, plan_segments, tp_slices
from verl_b200.parallel.zero import ZeroShardedParams


class _FakeZero:
    """Layout of a W-rank sharding computed without process groups."""

    def __init__(self, model, world):
        z = ZeroShardedParams([("", [("embed_tokens.weight", model.embed_tokens.weight), ("norm.weight", model.norm.weight)])]
                              + [(f"layers.{i}", l) for i, l in enumerate(model.layers)], work_dtype=torch.float32,
                              device="cpu", trainable=False)
        self.units = z.units
        full = {}
        for u in z.units:
            quantum = 256 * world
            u.padded = (u.numel + quantum - 1) // quantum * quantum
            u.shard = u.padded // world
        off = 0
        for u in z.units:
            u.offset = off
            off += u.shard
        self.total = off
        self.world = world
        # every rank's shard as bf16 bytes
        self.shards = []
        flat_units = []
        for u in z.units:
            flat = torch.zeros(u.padded, dtype=torch.bfloat16)
            for p, o, n in zip(u.params, u.offsets, u.numels):
                flat[o : o + n] = p.detach().reshape(-1).to(torch.bfloat16)
            flat_units.append(flat)
        for r in range(world):
            sh = torch.cat([f[r * u.shard : (r + 1) * u.shard] for f, u in zip(flat_units, z.units)])
            self.shards.append(sh.view(torch.uint8).numpy())


@pytest.mark.parametrize("world,tp", [(1, 1), (4, 1), (8, 2), (2, 2)])
def test_segment_table_reproduces_tp_slices(world, tp):
    torch.manual_seed(0)
    cfg = preset("tiny-qwen2", hidden_size=128, intermediate_size=256, num_attention_heads=4, num_key_value_heads=2, vocab_size=512)
    model = build_model(cfg, dtype=torch.float32)
    fz = _FakeZero(model, world)
    params = dict(model.named_parameters())
    for tp_rank in range(tp):
        dest, total = build_dest_layout(cfg, fz.units, tp_rank, tp)
        table = plan_segments(fz.units, world, dest)
        dst = np.zeros(total * 2, dtype=np.uint8)
        execute_on_host(table, fz.shards, dst)
        out = torch.from_numpy(dst).view(torch.bfloat16)
        for d in dest:
            p = params[d.name].detach().to(torch.bfloat16)
            rows = torch.cat([p[a:b] for a, b in d.row_ranges], dim=0) if p.dim() else p
            if d.col_range is not None:
                rows = rows[:, d.col_range[0] : d.col_range[1]]
            n = rows.numel()
            assert torch.equal(out[d.dst_off : d.dst_off + n].view(rows.shape), rows), d.name
        assert set(table["src_rank"].tolist()) <= set(range(world))
        assert (table["nbytes"] <= 1 << 20).all()


def test_tp_slices_of_fused_projections():
    cfg = preset("qwen2.5-7b")
    rr, cr = tp_slices(cfg, "layers.0.self_attn.qkv_proj.weight", (4608, 3584), 1, 2)
    assert rr == [(1792, 3584), (3584 + 256, 3584 + 512), (4096 + 256, 4096 + 512)] and cr is None
    rr, cr = tp_slices(cfg, "layers.0.mlp.gate_up_proj.weight", (37888, 3584), 0, 4)
    assert rr == [(0, 4736), (18944, 18944 + 4736)]
    rr, cr = tp_slices(cfg, "layers.0.mlp.down_proj.weight", (3584, 18944), 3, 4)
    assert rr == [(0, 3584)] and cr == (3 * 4736, 4 * 4736)
