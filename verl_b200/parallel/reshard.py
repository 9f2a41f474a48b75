"""Train -> rollout weight reshard: ZeRO flat shards to the rollout engine's (tensor-parallel) layout.

The trainer keeps, per unit (layer), 1/W of the unit's flattened parameters on every rank. The rollout
engine wants, per rank, either every full tensor (TP = 1) or its slice of every tensor: rows of
column-parallel weights (q / k / v parts of the fused qkv projection and gate / up parts of the fused MLP
input projection are sliced part by part, as ``default_tp_concat_fn`` in the reference regroups them,
verl/utils/megatron_utils.py:846), columns of row-parallel weights (o_proj, down_proj), everything else
replicated.

:func:`plan_segments` turns that into a table of (source rank, source byte offset, destination byte offset,
length) copies; ``PeerComm.segment_copy`` executes the whole table in ONE kernel launch that reads the
peers' shards over NVLink and writes the rollout weights in place. No NCCL call, no host staging, no
intermediate full tensor (the reference path is an all-gather per parameter, a copy into an IPC bucket and
two more copies on the inference side: verl/workers/fsdp_workers.py:677-756,
verl/workers/rollout/vllm_rollout/vllm_rollout.py:145-216).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from ..models.config import ModelConfig

SEG_DTYPE = np.dtype([("src_off", "<i8"), ("dst_off", "<i8"), ("nbytes", "<i8"), ("src_rank", "<i4"), ("pad", "<i4")])
MAX_SEG_BYTES = 1 << 20


@dataclass
class DestTensor:
    """Where one rollout tensor lives in the destination buffer and which part of the source parameter it is."""

    name: str
    dst_off: int  # elements from the start of the destination buffer
    shape: tuple
    row_ranges: list  # [(r0, r1), ...] rows of the source parameter, concatenated in this order
    col_range: Optional[tuple] = None  # (c0, c1) columns kept from each row (None = all)


def tp_model_config(cfg: ModelConfig, tp_rank: int, tp_size: int) -> ModelConfig:
    """Architecture of one tensor-parallel rank's slice of the model: 1 / tp of the query heads, of the KV heads (one
    replicated KV head per rank when there are fewer KV heads than ranks), of the MLP columns and of the experts."""
    import dataclasses

    if tp_size == 1:
        return cfg
    if not cfg.mlp_gated:
        raise ValueError(f"tensor parallelism is not implemented for the {cfg.model_type} MLP layout")
    Hq, Hk = cfg.num_attention_heads, cfg.num_key_value_heads
    if Hq % tp_size != 0:
        raise ValueError(f"tensor_model_parallel_size {tp_size} does not divide {Hq} attention heads")
    if Hk % tp_size != 0 and tp_size % Hk != 0:
        raise ValueError(f"tensor_model_parallel_size {tp_size} and {Hk} KV heads are incompatible")
    if not cfg.is_moe and cfg.intermediate_size % (8 * tp_size) != 0:
        raise ValueError(f"intermediate size {cfg.intermediate_size} cannot be split over {tp_size} ranks in multiples of 8")
    if cfg.is_moe and cfg.num_experts % tp_size != 0:
        raise ValueError(f"{cfg.num_experts} experts cannot be split over {tp_size} ranks")
    extra = dict(cfg.extra)
    extra.update({"tp_size": tp_size, "tp_rank": tp_rank})
    if cfg.is_moe:
        extra.update({"ep_size": tp_size, "ep_rank": tp_rank})
    return dataclasses.replace(cfg, num_attention_heads=Hq // tp_size, num_key_value_heads=max(Hk // tp_size, 1),
                               head_dim=cfg.head_dim, intermediate_size=cfg.intermediate_size // tp_size, extra=extra)


def tp_slices(cfg: ModelConfig, name: str, shape: tuple, tp_rank: int, tp_size: int, vocab_parallel_head: bool = False):
    """(row_ranges, col_range) of native parameter ``name`` owned by ``tp_rank`` (``cfg``: the whole model).
    ``vocab_parallel_head``: an untied ``lm_head.weight`` is split by vocabulary rows (training engine)."""
    rows = shape[0] if len(shape) >= 1 else 1
    if tp_size == 1 or len(shape) == 0:
        return [(0, rows)], None
    if vocab_parallel_head and name.endswith("lm_head.weight") and shape[0] % tp_size == 0:
        k = shape[0] // tp_size
        return [(tp_rank * k, (tp_rank + 1) * k)], None

    def part(r0, n):
        assert n % tp_size == 0, f"{name}: {n} rows not divisible by tp {tp_size}"
        k = n // tp_size
        return (r0 + tp_rank * k, r0 + (tp_rank + 1) * k)

    def kv_part(r0):
        Hk, D = cfg.num_key_value_heads, cfg.head_dim
        if Hk % tp_size == 0:
            return part(r0, Hk * D)
        head = tp_rank // (tp_size // Hk)  # fewer KV heads than ranks: neighbouring ranks share (replicate) a head
        return (r0 + head * D, r0 + (head + 1) * D)

    leaf = name.split(".")[-2] + "." + name.split(".")[-1] if "." in name else name
    if leaf in ("qkv_proj.weight", "qkv_proj.bias"):
        q, kv = cfg.q_size, cfg.kv_size
        return [part(0, q), kv_part(q), kv_part(q + kv)], None
    if leaf == "gate_up_proj.weight":
        i = shape[0] // 2
        return [part(0, i), part(i, i)], None
    if leaf in ("o_proj.weight", "down_proj.weight"):
        cols = shape[1]
        assert cols % tp_size == 0
        k = cols // tp_size
        return [(0, rows)], (tp_rank * k, (tp_rank + 1) * k)
    if leaf in ("mlp.gate_up_proj", "mlp.down_proj") and len(shape) == 3:  # stacked expert matrices: whole experts
        return [part(0, shape[0])], None
    return [(0, rows)], None


def shard_state_dict(cfg: ModelConfig, full: dict, tp_rank: int, tp_size: int, vocab_parallel_head: bool = False) -> dict:
    """This rank's slices of a whole-model state dict (native names), in the layout of :func:`tp_model_config`."""
    out = {}
    for name, t in full.items():
        row_ranges, col_range = tp_slices(cfg, name, tuple(t.shape), tp_rank, tp_size, vocab_parallel_head)
        if t.dim() == 0:
            out[name] = t
            continue
        piece = torch.cat([t[a:b] for a, b in row_ranges], dim=0) if len(row_ranges) > 1 or row_ranges[0] != (0, t.shape[0]) else t
        if col_range is not None:
            piece = piece[:, col_range[0] : col_range[1]]
        out[name] = piece.contiguous()
    return out


def unshard_state_dict(cfg: ModelConfig, parts: list, vocab_parallel_head: bool = False) -> dict:
    """Inverse of :func:`shard_state_dict`: the ranks' slices (rank order) -> whole tensors. Replicated tensors are
    taken from rank 0; replicated KV heads are de-duplicated."""
    tp = len(parts)
    if tp == 1:
        return dict(parts[0])
    out = {}
    for name, t0 in parts[0].items():
        leaf = name.split(".")[-2] + "." + name.split(".")[-1] if "." in name else name
        ts = [p[name] for p in parts]
        if leaf in ("qkv_proj.weight", "qkv_proj.bias"):
            Hq, Hk, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
            ql = Hq // tp * D
            kl = max(Hk // tp, 1) * D
            q = torch.cat([t[:ql] for t in ts], 0)
            step = 1 if Hk % tp == 0 else tp // Hk  # replicated heads: every `step`-th rank holds a new one
            k = torch.cat([t[ql : ql + kl] for t in ts[::step]], 0)
            v = torch.cat([t[ql + kl : ql + 2 * kl] for t in ts[::step]], 0)
            out[name] = torch.cat([q, k, v], 0)
        elif leaf == "gate_up_proj.weight":
            i = t0.shape[0] // 2
            out[name] = torch.cat([torch.cat([t[:i] for t in ts], 0), torch.cat([t[i:] for t in ts], 0)], 0)
        elif leaf in ("o_proj.weight", "down_proj.weight"):
            out[name] = torch.cat(ts, 1)
        elif leaf in ("mlp.gate_up_proj", "mlp.down_proj") and t0.dim() == 3:
            out[name] = torch.cat(ts, 0)
        elif vocab_parallel_head and name.endswith("lm_head.weight") and t0.shape[0] != cfg.vocab_size:
            out[name] = torch.cat(ts, 0)
        else:
            out[name] = t0
    return out


def build_dest_layout(cfg: ModelConfig, zero_units, tp_rank: int = 0, tp_size: int = 1, align: int = 8):
    """Destination layout: tensors back to back (16-byte aligned) in unit / parameter order."""
    out, off = [], 0
    for u in zero_units:
        for name, shape in zip(u.names, u.shapes):
            row_ranges, col_range = tp_slices(cfg, name, tuple(shape), tp_rank, tp_size)
            rows = sum(b - a for a, b in row_ranges)
            if len(shape) == 0:
                dshape = ()
            elif len(shape) == 1:
                dshape = (rows,)
            else:
                cols = shape[1] if col_range is None else col_range[1] - col_range[0]
                dshape = (rows, cols) + tuple(shape[2:])
            n = int(np.prod(dshape)) if dshape else 1
            out.append(DestTensor(name, off, dshape, row_ranges, col_range))
            off += (n + align - 1) // align * align
    return out, off


def plan_segments(zero_units, world: int, dest: list[DestTensor], elem_bytes: int = 2) -> np.ndarray:
    """Copy table for one destination rank. Source coordinates are byte offsets into a rank's ``shard16``."""
    segs = []
    by_name = {}
    for u in zero_units:
        for name, shape, o in zip(u.names, u.shapes, u.offsets):
            by_name[name] = (u, tuple(shape), o)

    def emit(u, flat_lo: int, n: int, dst_elem: int):
        """n contiguous elements of unit u's flat vector starting at flat_lo -> destination element dst_elem."""
        while n > 0:
            r = flat_lo // u.shard
            within = flat_lo - r * u.shard
            take = min(n, u.shard - within)
            done = 0
            while done < take:
                chunk = min(take - done, MAX_SEG_BYTES // elem_bytes)
                segs.append(((u.offset + within + done) * elem_bytes, (dst_elem + done) * elem_bytes, chunk * elem_bytes, r, 0))
                done += chunk
            flat_lo += take
            dst_elem += take
            n -= take

    for d in dest:
        u, shape, o = by_name[d.name]
        row_elems = int(np.prod(shape[1:])) if len(shape) > 1 else 1
        dst = d.dst_off
        if d.col_range is None:
            for (r0, r1) in d.row_ranges:
                n = (r1 - r0) * row_elems
                emit(u, o + r0 * row_elems, n, dst)
                dst += n
        else:
            c0, c1 = d.col_range
            inner = int(np.prod(shape[2:])) if len(shape) > 2 else 1
            width = (c1 - c0) * inner
            for (r0, r1) in d.row_ranges:
                for r in range(r0, r1):
                    emit(u, o + r * row_elems + c0 * inner, width, dst)
                    dst += width
    table = np.array(segs, dtype=SEG_DTYPE) if segs else np.zeros(0, dtype=SEG_DTYPE)
    bad = (table["src_off"] % 16 != 0) | (table["dst_off"] % 16 != 0) | (table["nbytes"] % 16 != 0)
    if bad.any():
        raise ValueError("reshard segments must be 16-byte aligned (tensor sizes / TP slices must be multiples of 8 elements)")
    return table


def execute_on_host(table: np.ndarray, shards: list[np.ndarray], dst: np.ndarray, elem_bytes: int = 2) -> None:
    """Reference execution of a segment table on host arrays (tests and the CPU path): ``shards[r]`` is rank r's
    flat shard viewed as bytes, ``dst`` the destination viewed as bytes."""
    for s in table:
        so, do, n, r = int(s["src_off"]), int(s["dst_off"]), int(s["nbytes"]), int(s["src_rank"])
        dst[do : do + n] = shards[r][so : so + n]


class RolloutWeights:
    """Destination buffer + copy table of one rollout rank, bound to the parameters of its model."""

    def __init__(self, cfg: ModelConfig, zero, model, tp_rank: int = 0, tp_size: int = 1):
        self.zero = zero
        self.dest, total = build_dest_layout(cfg, zero.units, tp_rank, tp_size)
        self.buffer = torch.zeros(total, dtype=zero.work_dtype, device=zero.device)
        own = dict(model.named_parameters())
        for d in self.dest:
            if d.name in own:
                n = int(np.prod(d.shape)) if d.shape else 1
                own[d.name].data = self.buffer[d.dst_off : d.dst_off + n].view(d.shape)
        table = plan_segments(zero.units, zero.world, self.dest, self.buffer.element_size())
        self.nseg = len(table)
        self.table_host = table
        self.table = torch.from_numpy(table.view(np.uint8).copy()).to(zero.device) if zero.device.type == "cuda" else None
        self.bytes_total = int(table["nbytes"].sum())
        self.bytes_remote = int(table["nbytes"][table["src_rank"] != zero.rank].sum())

    @torch.no_grad()
    def sync(self):
        z = self.zero
        if z.comm is not None and self.table is not None:
            z.comm.segment_copy(self.buffer, z.shard16, self.table, self.nseg)
            return
        # fallback: gather the shards with torch.distributed, then run the table locally
        import torch.distributed as dist

        if z.world > 1:
            parts = [torch.empty_like(z.shard16) for _ in range(z.world)]
            dist.all_gather(parts, z.shard16, group=z.group)
        else:
            parts = [z.shard16]
        eb = self.buffer.element_size()
        if z.world == 1:
            # one rank: the same source and destination views every time; one batched copy instead of a Python loop
            if getattr(self, "_views", None) is None or self._views[2] is not z.shard16:
                dst, src = [], []
                for s in self.table_host:
                    so, do, n = int(s["src_off"]) // eb, int(s["dst_off"]) // eb, int(s["nbytes"]) // eb
                    dst.append(self.buffer[do : do + n])
                    src.append(z.shard16[so : so + n])
                self._views = (dst, src, z.shard16)
            torch._foreach_copy_(self._views[0], self._views[1])
            return
        for s in self.table_host:
            so, do, n, r = int(s["src_off"]) // eb, int(s["dst_off"]) // eb, int(s["nbytes"]) // eb, int(s["src_rank"])
            self.buffer[do : do + n].copy_(parts[r][so : so + n])
