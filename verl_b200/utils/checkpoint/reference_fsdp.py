"""Interchange with shard files written by torch FSDP, the format of the reference's checkpoints.

The reference saves ``model.state_dict()`` of an FSDP-wrapped HF model per rank as
``model_world_size_{W}_rank_{r}.pt`` (verl/utils/checkpoint/fsdp_checkpoint_manager.py:219-226): HF parameter names,
values that are ``DTensor`` (FSDP2 and FSDP1 with ``use_orig_params``; placement ``Shard(0)`` on a 1-D mesh, or
``(Replicate, Shard(0))`` under HSDP) or ``ShardedTensor`` (older FSDP1). Its merger re-assembles them by concatenating
the local tensors along the sharded dimension (verl/model_merger/fsdp_model_merger.py:115-264).

* :func:`load_reference_fsdp_shards` does that re-assembly and maps the HF names to this package's fused layout, so
  that a checkpoint directory written by the reference can be resumed from or merged here;
* :func:`save_reference_fsdp_shards` writes this engine's weights as ``Shard(0)`` DTensor state dicts under HF names,
  which the reference's loader and merger read (``checkpoint.save_contents`` entry ``"fsdp_model"``).
"""

from __future__ import annotations

import json
from pathlib import Path

import torch
import torch.distributed as dist


def _local_and_placement(v):
    """(local tensor, shard dim | None, shard index | None) of one state-dict value."""
    try:
        from torch.distributed.tensor import DTensor, Shard
    except Exception:  # pragma: no cover
        DTensor, Shard = (), None
    if DTensor and isinstance(v, DTensor):
        dim = None
        for pl in v.placements:
            if isinstance(pl, Shard):
                dim = pl.dim
        return v._local_tensor, dim, None
    if hasattr(v, "local_shards") and hasattr(v, "metadata"):  # ShardedTensor of FSDP1
        shards = v.local_shards()
        if not shards:
            return torch.empty(0), 0, None
        off = shards[0].metadata.shard_offsets
        dim = next((i for i, o in enumerate(off) if o != 0), 0)
        return shards[0].tensor, dim, off[dim]
    return v, None, None


def merge_reference_state_dicts(states: list[dict], mesh_shape: tuple | None = None) -> dict:
    """Full HF-named tensors from the per-rank state dicts (rank order). Under HSDP (``mesh_shape = (replicas,
    shards)``) only the first replica's ranks are used."""
    W = len(states)
    shards = W if not mesh_shape or len(mesh_shape) == 1 else int(mesh_shape[-1])
    out = {}
    for key in states[0].keys():
        parts = [_local_and_placement(st[key]) for st in states[:shards]]
        local0, dim, _ = parts[0]
        if not isinstance(local0, torch.Tensor):
            continue
        if dim is None:
            out[key] = local0.clone()
            continue
        if parts[0][2] is not None:  # ShardedTensor: order by recorded offset
            parts = sorted(parts, key=lambda p: p[2] if p[2] is not None else 0)
        out[key] = torch.cat([p[0] for p in parts if p[0].numel()], dim=dim).contiguous()
    return out


def load_reference_fsdp_shards(path: str | Path, model_config=None) -> dict:
    """Directory of torch-FSDP shard files -> full tensors under this package's parameter names."""
    from ...models.config import ModelConfig
    from ...models.hf_io import hf_to_native_state_dict

    path = Path(path)
    meta = json.loads((path / "fsdp_config.json").read_text()) if (path / "fsdp_config.json").exists() else {}
    files = sorted(path.glob("model_world_size_*_rank_*.pt"), key=lambda f: int(f.stem.rsplit("_", 1)[1]))
    if not files:
        raise FileNotFoundError(f"no model_world_size_*_rank_*.pt under {path}")
    W = int(meta.get("world_size", len(files)))
    states = [torch.load(path / f"model_world_size_{W}_rank_{r}.pt", map_location="cpu", weights_only=False)
              for r in range(W)]
    if not isinstance(states[0], dict) or "format" in states[0]:
        raise ValueError(f"{files[0].name} is not a torch-FSDP state dict (supported: this engine's flat shards, "
                         "DTensor / ShardedTensor state dicts, or HF safetensors under huggingface/)")
    mesh_shape = None
    for v in states[0].values():
        mesh = getattr(v, "device_mesh", None)
        if mesh is not None:
            mesh_shape = tuple(mesh.mesh.shape)
            break
    hf = merge_reference_state_dicts(states, mesh_shape)
    if model_config is None:
        model_config = ModelConfig.from_pretrained(path / "huggingface")
    return hf_to_native_state_dict(model_config, hf)


def save_reference_fsdp_shards(engine, local_path: str | Path) -> None:
    """Write ``model_world_size_{W}_rank_{r}.pt`` as the reference's FSDP2 engine does: HF names, every parameter a
    DTensor sharded on dim 0 over the data-parallel group (``torch.chunk`` boundaries, empty trailing shards allowed).
    Collective: every rank of the engine calls it (the full tensors are gathered one by one)."""
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import DTensor, Shard

    from ...models.hf_io import native_to_hf_items

    z = engine.zero
    W, r = z.world, z.rank
    path = Path(local_path)
    path.mkdir(parents=True, exist_ok=True)
    mesh = None
    if dist.is_initialized():
        mesh = init_device_mesh(z.device.type if z.device.type == "cuda" else "cpu", (dist.get_world_size(z.group),),
                                mesh_dim_names=("fsdp",)) if z.world == dist.get_world_size() else None
    sd = {}
    named = engine._merged_named_tensors() if hasattr(engine, "_merged_named_tensors") else z.named_full_tensors()
    for name, full in native_to_hf_items(engine.model_config, named):
        full = full.detach()
        if full.dim() == 0 or mesh is None:
            sd[name] = full.cpu().clone()
            continue
        chunks = list(torch.chunk(full, W, dim=0))
        local = chunks[r] if r < len(chunks) else full.new_empty((0,) + tuple(full.shape[1:]))
        sd[name] = DTensor.from_local(local.cpu().clone() if mesh.device_type == "cpu" else local.clone(), mesh, [Shard(0)],
                                      run_check=False, shape=full.shape, stride=full.stride())
    torch.save(sd, path / f"model_world_size_{W}_rank_{r}.pt")
    if r == 0:
        (path / "fsdp_config.json").write_text(json.dumps({"FSDP_version": 2, "world_size": W}, indent=4))
        engine.model_config.save_pretrained(path / "huggingface")
    if dist.is_initialized():
        dist.barrier(group=z.group)
