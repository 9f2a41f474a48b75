"""Merge a sharded training checkpoint into a HuggingFace directory.

    python -m verl_b200.model_merger merge --backend fsdp --local_dir ckpt/global_step_10/actor --target_dir out/hf
    python -m verl_b200.model_merger test  --backend fsdp --local_dir ckpt/global_step_10/actor --test_hf_dir out/hf

Role of verl/model_merger/ (``merge|test --backend fsdp|megatron --local_dir --target_dir``): the FSDP merger
there concatenates DTensor shards by placement; here every rank file stores, per parameter, the slice of the flat
unit shard that belongs to it (``model_world_size_{W}_rank_{r}.pt``), so merging is a scatter by (start, length).
Directories written by the reference itself (torch FSDP: per-parameter DTensor / ShardedTensor shards in the same
file names) are recognised by their content and merged by placement, so the CLI serves both. ``--backend megatron``
is accepted for CLI compatibility and handled the same way: the engine writes one format whatever its parallel layout
(tensor-, pipeline- and expert-parallel runs export merged tensors).
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from ..models.config import ModelConfig
from ..models.hf_io import load_hf_checkpoint, native_to_hf_state_dict, save_hf_checkpoint
from ..utils.checkpoint.native_checkpoint import merge_sharded_checkpoint


def merge_checkpoint(local_dir: str, target_dir: str, dtype: torch.dtype = torch.bfloat16, tie_word_embedding: bool = False) -> dict:
    local = Path(local_dir)
    cfg = ModelConfig.from_pretrained(local / "huggingface")
    sd = merge_sharded_checkpoint(local)
    if tie_word_embedding:
        sd.pop("lm_head.weight", None)
    save_hf_checkpoint(cfg, sd, target_dir, dtype=dtype)
    # tokenizer / generation files saved next to the config travel with the merged model
    for extra in (local / "huggingface").glob("*"):
        if extra.name not in ("config.json",) and extra.suffix in (".json", ".txt", ".model", ".jinja") and not (Path(target_dir) / extra.name).exists():
            (Path(target_dir) / extra.name).write_bytes(extra.read_bytes())
    return sd


def test_merged(local_dir: str, test_hf_dir: str, atol: float = 1e-6) -> None:
    """Every merged tensor equals the tensor of the same HF name in ``test_hf_dir`` (after the bf16 cast)."""
    cfg = ModelConfig.from_pretrained(Path(local_dir) / "huggingface")
    merged = native_to_hf_state_dict(cfg, merge_sharded_checkpoint(local_dir))
    _, ref_native = load_hf_checkpoint(test_hf_dir)
    ref = native_to_hf_state_dict(cfg, ref_native)
    missing = set(ref) ^ set(merged)
    if missing:
        raise AssertionError(f"key mismatch between merged and reference model: {sorted(missing)[:8]}")
    for k, v in merged.items():
        a, b = v.to(torch.bfloat16).float(), ref[k].to(torch.bfloat16).float()
        if a.shape != b.shape:
            raise AssertionError(f"{k}: shape {tuple(a.shape)} vs {tuple(b.shape)}")
        if not torch.allclose(a, b, atol=atol, rtol=1e-5):
            raise AssertionError(f"{k}: max abs diff {(a - b).abs().max().item():.3e}")


def main(argv=None):
    ap = argparse.ArgumentParser(prog="verl_b200.model_merger")
    sub = ap.add_subparsers(dest="operation", required=True)
    for name in ("merge", "test"):
        p = sub.add_parser(name)
        p.add_argument("--backend", choices=["fsdp", "megatron", "native"], default="fsdp")
        p.add_argument("--local_dir", required=True)
        p.add_argument("--tie-word-embedding", action="store_true")
        p.add_argument("--trust-remote-code", action="store_true")
        p.add_argument("--use_cpu_initialization", action="store_true")
        if name == "merge":
            p.add_argument("--target_dir", default="tmp")
            p.add_argument("--hf_upload_path", default=None)
            p.add_argument("--private", action="store_true")
        else:
            p.add_argument("--test_hf_dir", required=True)
    a = ap.parse_args(argv)
    if a.operation == "merge":
        merge_checkpoint(a.local_dir, a.target_dir, tie_word_embedding=a.tie_word_embedding)
        if a.hf_upload_path:
            print("[model_merger] hub upload skipped: no network access from this process")
        print(json.dumps({"merged_to": a.target_dir}))
    else:
        test_merged(a.local_dir, a.test_hf_dir)
        print(json.dumps({"test": "ok"}))


if __name__ == "__main__":
    main()
