"""LoRA adapters on the native decoder (role of ``peft.get_peft_model`` + the LoRA branches of
verl/workers/fsdp_workers.py:_build_model_optimizer and verl/utils/fsdp_utils.py:569-669).

A target ``Linear`` computes ``y = x W^T + (alpha / r) * (x A^T) B^T`` with ``A [r, in]`` (Kaiming-uniform) and
``B [out, r]`` (zero), both fp32 and cast to the activation dtype at use. The base weights are frozen: under LoRA the
engine keeps no fp32 master, moments or gradients for them. The adapter tensors are NOT registered as module
parameters (they must stay out of the ZeRO flat shards); every rank holds a full replica and gradients are summed
over the data-parallel group.

Module names follow the fused layout of this model: ``qkv_proj`` (HF: q_proj, k_proj, v_proj), ``o_proj``,
``gate_up_proj`` (HF: gate_proj, up_proj), ``down_proj``. ``target_modules`` accepts HF names and maps them.
"""

from __future__ import annotations

import json
import math
import os
import re
from typing import Iterable, Optional

import torch
import torch.nn as nn

_HF_TO_FUSED = {"q_proj": "qkv_proj", "k_proj": "qkv_proj", "v_proj": "qkv_proj", "gate_proj": "gate_up_proj",
                "up_proj": "gate_up_proj", "o_proj": "o_proj", "down_proj": "down_proj", "qkv_proj": "qkv_proj",
                "gate_up_proj": "gate_up_proj"}
_ALL_LINEAR = ("qkv_proj", "o_proj", "gate_up_proj", "down_proj")


def _wanted(name: str, targets, exclude) -> bool:
    leaf = name.rsplit(".", 1)[-1]
    if exclude:
        ex = [exclude] if isinstance(exclude, str) else list(exclude)
        if any(re.fullmatch(e, name) or leaf == _HF_TO_FUSED.get(e, e) for e in ex):
            return False
    if targets in (None, "all-linear", "all_linear"):
        return leaf in _ALL_LINEAR
    if isinstance(targets, str):
        return re.fullmatch(targets, name) is not None or leaf == _HF_TO_FUSED.get(targets, targets)
    return leaf in {_HF_TO_FUSED.get(t, t) for t in targets}


def apply_lora(model: nn.Module, rank: int, alpha: float = 16.0, target_modules="all-linear", exclude_modules=None,
               seed: int = 0) -> list[str]:
    """Attach adapters to the matching ``Linear`` modules of ``model.layers``. Returns the adapted module names."""
    from .transformer import Linear

    g = torch.Generator().manual_seed(10_000 + seed)
    names = []
    for name, mod in model.named_modules():
        if not isinstance(mod, Linear) or not name.startswith("layers.") or not _wanted(name, target_modules, exclude_modules):
            continue
        out_f, in_f = mod.weight.shape
        dev = mod.weight.device
        a = torch.empty(rank, in_f)
        bound = 1.0 / math.sqrt(in_f)  # kaiming_uniform_(a=sqrt(5)) on [r, in]
        a.uniform_(-bound, bound, generator=g)
        # plain attributes: keeps them out of named_parameters() and so out of the ZeRO flat shards
        mod.__dict__["lora_A"] = nn.Parameter(a.to(dev))
        mod.__dict__["lora_B"] = nn.Parameter(torch.zeros(out_f, rank, device=dev))
        mod.__dict__["lora_scale"] = float(alpha) / rank
        names.append(name)
    model.__dict__["lora_modules"] = names
    return names


def lora_named_parameters(model: nn.Module) -> Iterable[tuple[str, nn.Parameter]]:
    mods = dict(model.named_modules())
    for name in getattr(model, "lora_modules", []):
        yield name + ".lora_A", mods[name].lora_A
        yield name + ".lora_B", mods[name].lora_B


def lora_delta(mod) -> torch.Tensor:
    """``(alpha / r) * B A`` in fp32, the matrix to add to the module's weight. On the GPU the product runs on the
    framework's own GEMM with the adapters rounded to bf16, exactly what the forward pass multiplies with."""
    a, b = mod.lora_A.detach(), mod.lora_B.detach()
    if a.is_cuda:
        from .. import ops

        prod = ops.gemm(b.to(torch.bfloat16), a.to(torch.bfloat16).contiguous(), b_mn=True, out_dtype=torch.float32)
        return mod.lora_scale * prod
    return mod.lora_scale * (b.float() @ a.float())


@torch.no_grad()
def merge_lora_into(src_model: nn.Module, dst_model: nn.Module) -> int:
    """dst.W += delta for every adapted module of ``src_model`` (``dst_model``: a model with the same module names
    whose weights currently equal the base weights, e.g. the rollout copy right after a weight sync)."""
    src, dst = dict(src_model.named_modules()), dict(dst_model.named_modules())
    n = 0
    for name in getattr(src_model, "lora_modules", []):
        w = dst[name].weight
        w.add_(lora_delta(src[name]).to(device=w.device, dtype=w.dtype))
        n += 1
    return n


def peft_config(model_cfg, rank: int, alpha: float, target_modules) -> dict:
    return {"peft_type": "LORA", "task_type": "CAUSAL_LM", "r": int(rank), "lora_alpha": float(alpha), "lora_dropout": 0.0,
            "bias": "none", "target_modules": ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]
            if target_modules in (None, "all-linear", "all_linear") else target_modules, "fused_layout": "verl_b200"}


def save_adapter(model: nn.Module, path: str, rank: int, alpha: float, target_modules=None) -> None:
    """``adapter_config.json`` + ``adapter_model.safetensors`` with HF/PEFT-style names split per HF projection:
    the fused ``qkv_proj`` adapter shares A between q/k/v and splits the rows of B."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    cfg = model.cfg if hasattr(model, "cfg") else None
    out = {}
    mods = dict(model.named_modules())
    for name in getattr(model, "lora_modules", []):
        m = mods[name]
        a, b = m.lora_A.detach().float().cpu(), m.lora_B.detach().float().cpu()
        prefix, leaf = name.rsplit(".", 1)
        base = f"base_model.model.model.{prefix}"
        if leaf == "qkv_proj" and cfg is not None:
            q = cfg.num_attention_heads * cfg.head_dim
            kv = cfg.num_key_value_heads * cfg.head_dim
            for nm, lo, hi in (("q_proj", 0, q), ("k_proj", q, q + kv), ("v_proj", q + kv, q + 2 * kv)):
                out[f"{base}.{nm}.lora_A.weight"], out[f"{base}.{nm}.lora_B.weight"] = a.clone(), b[lo:hi].clone()
        elif leaf == "gate_up_proj":
            half = b.shape[0] // 2
            for nm, lo, hi in (("gate_proj", 0, half), ("up_proj", half, 2 * half)):
                out[f"{base}.{nm}.lora_A.weight"], out[f"{base}.{nm}.lora_B.weight"] = a.clone(), b[lo:hi].clone()
        else:
            out[f"{base}.{leaf}.lora_A.weight"], out[f"{base}.{leaf}.lora_B.weight"] = a, b
    save_file({k: v.contiguous() for k, v in out.items()}, os.path.join(path, "adapter_model.safetensors"))
    with open(os.path.join(path, "adapter_config.json"), "w") as f:
        json.dump(peft_config(cfg, rank, alpha, target_modules), f, indent=2)


def lora_state_dict(model: nn.Module) -> dict:
    return {k: v.detach().cpu().clone() for k, v in lora_named_parameters(model)}


@torch.no_grad()
def load_lora_state_dict(model: nn.Module, state: dict) -> None:
    for k, p in lora_named_parameters(model):
        p.copy_(state[k].to(p.device))
