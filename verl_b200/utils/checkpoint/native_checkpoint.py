"""Sharded checkpoints in the verl FSDP layout plus HuggingFace export.

Directory layout written / read (verl/utils/checkpoint/fsdp_checkpoint_manager.py:56-362,
docs/advance/checkpoint.rst:20-62):

    <dir>/model_world_size_{W}_rank_{r}.pt        this rank's parameter shard
    <dir>/optim_world_size_{W}_rank_{r}.pt        this rank's optimizer shard (fp32 master + Adam moments)
    <dir>/extra_state_world_size_{W}_rank_{r}.pt  lr-scheduler step + RNG state
    <dir>/fsdp_config.json                        {"FSDP_version": 2, "world_size": W, "shard_format": ...}
    <dir>/huggingface/                            config.json (always) + safetensors when "hf_model" is saved

The reference stores ``DTensor`` shards produced by torch FSDP. This engine shards flat per-layer vectors
instead, so by default the model file holds, per parameter, the slice of the flattened tensor this rank owns
together with (global shape, start offset, length) and ``shard_format`` names that layout;
:func:`merge_sharded_checkpoint` re-assembles full tensors from the W files (the job of
``python -m verl.model_merger merge --backend fsdp``). Both directions of interchange with the reference go
through :mod:`.reference_fsdp`: directories written by torch FSDP load and merge here, and the save content
``"fsdp_model"`` (instead of ``"model"``) writes torch-FSDP-style DTensor shard files.
"""

from __future__ import annotations

import json
import os
import random
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

from ...models.hf_io import save_hf_checkpoint

FLAT_SHARD_FORMAT = "verl_b200.flat_shard.v1"


def _rng_state() -> dict:
    st = {"cpu": torch.get_rng_state(), "numpy": np.random.get_state(), "random": random.getstate()}
    if torch.cuda.is_available():
        st["cuda"] = torch.cuda.get_rng_state()
    return st


def _load_rng_state(st: dict) -> None:
    torch.set_rng_state(st["cpu"])
    np.random.set_state(st["numpy"])
    random.setstate(st["random"])
    if torch.cuda.is_available() and "cuda" in st:
        torch.cuda.set_rng_state(st["cuda"])


def _param_slices(zero, flat: torch.Tensor) -> dict:
    """{param name: {"shape", "start", "data"}} — the part of each flattened parameter held by this rank."""
    out = {}
    for u in zero.units:
        lo, hi = zero.rank * u.shard, (zero.rank + 1) * u.shard
        for name, p_shape, o in zip(u.names, u.shapes, u.offsets):
            n = int(np.prod(p_shape)) if len(p_shape) else 1
            s, e = max(o, lo), min(o + n, hi)
            if s >= e:
                out[name] = {"shape": p_shape, "start": 0, "data": flat.new_empty(0)}
                continue
            out[name] = {"shape": p_shape, "start": s - o,
                         "data": flat[u.offset + s - lo : u.offset + e - lo].detach().cpu().clone()}
    return out


def save_engine_checkpoint(engine, local_path: str, global_step: int = 0,
                           save_contents=("model", "optimizer", "extra")) -> None:
    z = engine.zero
    path = Path(local_path)
    if z.rank == 0:
        path.mkdir(parents=True, exist_ok=True)
    if dist.is_initialized():
        dist.barrier()
    W, r = _file_world_rank(engine)
    if getattr(engine, "hsdp", False) and getattr(engine, "replica_index", 0) != 0:
        # hybrid sharding: the replicas hold identical shards; the first replica group writes the files
        if dist.is_initialized():
            dist.barrier()
        return
    if "fsdp_model" in save_contents:
        # torch-FSDP shard files (HF names, dim-0 DTensor shards): what the reference's loader and merger read
        from .reference_fsdp import save_reference_fsdp_shards

        save_reference_fsdp_shards(engine, path)
    elif "model" in save_contents:
        src = z.master if z.trainable else z.shard16
        layout = int(getattr(engine, "tp_size", 1)) * 1000 + int(getattr(engine, "pp_size", 1))
        torch.save({"format": FLAT_SHARD_FORMAT, "world_size": W, "rank": r, "tp": layout if layout != 1001 else 1,
                    "layout": _layout_sig(z),
                    "params": _param_slices(z, src)},
                   path / f"model_world_size_{W}_rank_{r}.pt")
    if "optimizer" in save_contents and z.trainable:
        torch.save({"format": FLAT_SHARD_FORMAT, "world_size": W, "rank": r, "step": engine.step_count, "layout": _layout_sig(z),
                    "exp_avg": _param_slices(z, z.exp_avg), "exp_avg_sq": _param_slices(z, z.exp_avg_sq)},
                   path / f"optim_world_size_{W}_rank_{r}.pt")
    if "extra" in save_contents:
        torch.save({"lr_scheduler": {"lr_step": engine.lr_step, "step_count": engine.step_count}, "rng": _rng_state(),
                    "global_step": global_step}, path / f"extra_state_world_size_{W}_rank_{r}.pt")
    if getattr(engine, "_lora_params", None) and r == 0:
        # LoRA: the base weights above are frozen; the adapter (PEFT layout) and its optimizer state live beside them
        from ...models.lora import lora_state_dict, save_adapter

        lo = engine.lora
        save_adapter(engine.model, str(path / "lora_adapter"), int(lo["rank"]), float(lo.get("alpha", 16) or 16),
                     lo.get("target_modules"))
        torch.save({"lora": lora_state_dict(engine.model), "optimizer": engine._lora_opt.state_dict(),
                    "step": engine.step_count}, path / "lora_train_state.pt")
    if r == 0:
        fmt = "torch.fsdp.dtensor" if "fsdp_model" in save_contents else FLAT_SHARD_FORMAT
        (path / "fsdp_config.json").write_text(json.dumps({"FSDP_version": 2, "world_size": W, "shard_format": fmt}, indent=4))
        hf_dir = path / "huggingface"
        hf_dir.mkdir(exist_ok=True)
        engine.model_config.save_pretrained(hf_dir)
    if "hf_model" in save_contents:
        sd = {}
        named = engine._merged_named_tensors() if hasattr(engine, "_merged_named_tensors") else z.named_full_tensors()
        for k, v in named:  # collective: every rank takes part in the gathers (LoRA: merged weights)
            if r == 0:
                sd[k] = v.detach().to(torch.bfloat16).cpu()
        if r == 0:
            save_hf_checkpoint(engine.model_config, sd, path / "huggingface")
    if dist.is_initialized():
        dist.barrier()


def _restore(zero, dst: torch.Tensor, slices: dict) -> None:
    for u in zero.units:
        lo, hi = zero.rank * u.shard, (zero.rank + 1) * u.shard
        for name, o in zip(u.names, u.offsets):
            ent = slices[name]
            data = ent["data"]
            if data.numel() == 0:
                continue
            s = o + ent["start"]
            dst[u.offset + s - lo : u.offset + s - lo + data.numel()].copy_(data.to(dst.device, dst.dtype))


def _layout_sig(zero) -> str:
    """Fingerprint of how the parameters are cut into shards: per-rank slices can be restored directly only into the
    same cut (another unit composition, e.g. expert-parallel units, goes through the full tensors)."""
    import hashlib

    h = hashlib.sha1()
    for u in zero.units:
        h.update(f"{u.name}|{','.join(u.names)}|{u.shard}|{u.padded};".encode())
    return h.hexdigest()[:16]


def _file_world_rank(engine) -> tuple[int, int]:
    """(W, r) in the shard file names: the sharding group's, or (tensor parallelism: one set of slices per
    tensor-parallel rank) the engine group's."""
    if getattr(engine, "tp_size", 1) > 1 or getattr(engine, "pp_size", 1) > 1:
        return engine.full_world, engine.full_rank
    return engine.zero.world, engine.zero.rank


def load_engine_checkpoint(engine, local_path: str, load_contents=("model", "optimizer", "extra")) -> None:
    z = engine.zero
    path = Path(local_path)
    W, r = _file_world_rank(engine)
    mfile = path / f"model_world_size_{W}_rank_{r}.pt"
    if "model" in load_contents:
        st = torch.load(mfile, map_location="cpu", weights_only=False) if mfile.exists() else None
        tp = int(getattr(engine, "tp_size", 1)) * 1000 + int(getattr(engine, "pp_size", 1))  # (tp, pp) of the layout
        tp = tp if tp != 1001 else 1
        if (isinstance(st, dict) and st.get("format") == FLAT_SHARD_FORMAT and st["world_size"] == W and st.get("tp", 1) == tp
                and st.get("layout", _layout_sig(z)) == _layout_sig(z)):
            if z.trainable:
                _restore(z, z.master, st["params"])
                z.shard16.copy_(z.master.to(z.shard16.dtype))
            else:
                _restore(z, z.shard16, st["params"])
        elif tp > 1:
            raise ValueError(f"{path}: a tensor- / pipeline-parallel engine resumes from shard files of the same layout "
                             f"(world {W}) or from the HF weights under huggingface/ (model.path)")
        else:
            # another world size, or shard files written by torch FSDP (the reference's DTensor / ShardedTensor state
            # dicts): rebuild full tensors from all files of the directory and re-shard them
            z.load_full_state(merge_sharded_checkpoint(path, engine.model_config))
    ofile = path / f"optim_world_size_{W}_rank_{r}.pt"
    if "optimizer" in load_contents and z.trainable:
        st = torch.load(ofile, map_location="cpu", weights_only=False) if ofile.exists() else None
        if isinstance(st, dict) and st.get("format") == FLAT_SHARD_FORMAT and st.get("layout", _layout_sig(z)) == _layout_sig(z):
            _restore(z, z.exp_avg, st["exp_avg"])
            _restore(z, z.exp_avg_sq, st["exp_avg_sq"])
            engine.step_count = int(st.get("step", 0))
        elif r == 0:
            why = ("was written by another engine" if st is not None else
                   f"is absent (the checkpoint has another world size than {W}, or was saved without the optimizer)")
            print(f"[verl_b200] WARNING: {ofile.name} {why}: Adam moments restart from zero, "
                  "the parameters and the learning-rate schedule are restored")
    lfile = path / "lora_train_state.pt"
    if getattr(engine, "_lora_params", None) and lfile.exists():
        from ...models.lora import load_lora_state_dict

        st = torch.load(lfile, map_location="cpu", weights_only=False)
        if "model" in load_contents:
            load_lora_state_dict(engine.model, st["lora"])
        if "optimizer" in load_contents:
            engine._lora_opt.load_state_dict(st["optimizer"])
            engine.step_count = int(st.get("step", 0))
    efile = path / f"extra_state_world_size_{W}_rank_{r}.pt"
    if "extra" in load_contents and efile.exists():
        st = torch.load(efile, map_location="cpu", weights_only=False)
        engine.lr_step = int(st["lr_scheduler"]["lr_step"])
        engine.step_count = int(st["lr_scheduler"].get("step_count", engine.step_count))
        _load_rng_state(st["rng"])


def merge_sharded_checkpoint(local_path: str | Path, model_config=None) -> dict:
    """Re-assemble full (native-named) tensors from all ``model_world_size_*_rank_*.pt`` files of a directory: this
    engine's flat shards, or the per-parameter DTensor / ShardedTensor shards torch FSDP writes in the reference
    (those need ``model_config``, or the ``huggingface/config.json`` of the directory, for the name mapping)."""
    path = Path(local_path)
    cfg = json.loads((path / "fsdp_config.json").read_text())
    W = int(cfg["world_size"])
    first = torch.load(path / f"model_world_size_{W}_rank_0.pt", map_location="cpu", weights_only=False)
    if not (isinstance(first, dict) and first.get("format") == FLAT_SHARD_FORMAT):
        from .reference_fsdp import load_reference_fsdp_shards

        return load_reference_fsdp_shards(path, model_config)
    full: dict = {}
    for r in range(W):
        st = first if r == 0 else torch.load(path / f"model_world_size_{W}_rank_{r}.pt", map_location="cpu",
                                             weights_only=False)
        for name, ent in st["params"].items():
            n = int(np.prod(ent["shape"])) if len(ent["shape"]) else 1
            if name not in full:
                full[name] = torch.zeros(n, dtype=ent["data"].dtype if ent["data"].numel() else torch.float32)
            d = ent["data"]
            if d.numel():
                if full[name].dtype != d.dtype:
                    full[name] = full[name].to(d.dtype)
                full[name][ent["start"] : ent["start"] + d.numel()] = d
            full[name + "//shape"] = ent["shape"]
    out = {}
    for k in [k for k in full if not k.endswith("//shape")]:
        out[k] = full[k].view(full[k + "//shape"])
    return out
