"""Model helpers (subset of verl/utils/model.py that has a meaning without HF model classes / Megatron)."""

from __future__ import annotations

import json
import os

import torch
import torch.nn as nn


def update_model_config(module_config, override_config_kwargs: dict) -> None:
    """verl/utils/model.py:61-71: recursive setattr of overrides."""
    for k, v in (override_config_kwargs or {}).items():
        if isinstance(v, dict) and hasattr(module_config, k) and not isinstance(getattr(module_config, k), dict):
            update_model_config(getattr(module_config, k), v)
        else:
            setattr(module_config, k, v)


def get_model_size(model: nn.Module, scale: str = "auto"):
    """verl/utils/model.py:149-173."""
    n = sum(p.numel() for p in model.parameters())
    if scale == "auto":
        scale = "B" if n > 1e9 else "M" if n > 1e6 else "K" if n > 1e3 else ""
    div = {"B": 1e9, "M": 1e6, "K": 1e3, "": 1}[scale]
    return n / div, scale


def print_model_size(model: nn.Module, name: str | None = None) -> None:
    n, scale = get_model_size(model)
    print(f"{name or model.__class__.__name__} contains {n:.2f}{scale} parameters")


def compute_position_id_with_mask(mask: torch.Tensor) -> torch.Tensor:
    """verl/utils/model.py:226-227."""
    return torch.clip(torch.cumsum(mask, dim=-1) - 1, min=0, max=None)


def create_random_mask(input_ids: torch.Tensor, max_ratio_of_valid_token: float, max_ratio_of_left_padding: float,
                       min_ratio_of_valid_token: float = 0.0) -> torch.Tensor:
    """Random left/right padded attention mask for tests (verl/utils/model.py:183-223)."""
    assert 0 < max_ratio_of_valid_token <= 1 and 0 <= max_ratio_of_left_padding < 1
    b, s = input_ids.shape
    max_valid = max(1, int(s * max_ratio_of_valid_token))
    min_valid = max(1, int(s * min_ratio_of_valid_token))
    max_left = int(s * max_ratio_of_left_padding)
    assert max_valid + max_left <= s
    mask = torch.ones_like(input_ids, dtype=torch.int64)
    for i in range(b):
        left = int(torch.randint(0, max_left + 1, (1,)))
        valid = int(torch.randint(min_valid, max_valid + 1, (1,)))
        mask[i, :left] = 0
        mask[i, left + valid:] = 0
    return mask


def pad_packed_inputs(unpad_tokens: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen_in_batch: int, size: int):
    """Pad a packed stream to a multiple of ``size`` with one extra dummy sequence (verl/utils/model.py:503-533)."""
    total = unpad_tokens.shape[0]
    pad = (-total) % size
    if pad:
        if unpad_tokens.ndim == 1:
            unpad_tokens = torch.nn.functional.pad(unpad_tokens, (0, pad))
        else:
            unpad_tokens = torch.nn.functional.pad(unpad_tokens, (0, 0, 0, pad))
        cu_seqlens = torch.nn.functional.pad(cu_seqlens, (0, 1), value=int(cu_seqlens[-1]) + pad)
        max_seqlen_in_batch = max(max_seqlen_in_batch, pad)
    return unpad_tokens, cu_seqlens, max_seqlen_in_batch


def get_lora_rank_from_adapter(adapter_path: str | os.PathLike) -> int:
    """verl/utils/model.py:741-774: read ``r`` from a PEFT adapter_config.json."""
    path = os.path.join(adapter_path, "adapter_config.json")
    if not os.path.exists(path):
        raise FileNotFoundError(f"adapter_config.json not found in {adapter_path}")
    with open(path) as f:
        cfg = json.load(f)
    if "r" not in cfg:
        raise ValueError("LoRA rank 'r' not found in adapter_config.json")
    return int(cfg["r"])


def check_target_modules(config, key: str) -> bool:
    """PEFT-style target-module match (verl/utils/model.py:274-322): str = full regex, list = suffix match."""
    import re

    target = config.target_modules if hasattr(config, "target_modules") else config["target_modules"]
    if isinstance(target, str):
        return re.fullmatch(target, key) is not None
    return any(key == t or key.endswith("." + t) for t in target)


def convert_weight_keys(state_dict: dict, model=None) -> dict:
    """Checkpoints saved by other tool chains prefix or rename keys (``_checkpoint_conversion_mapping`` of HF models,
    verl/utils/model.py:230-248). The native model takes HF names through ``models.hf_io``; what is left to undo
    here are wrapper prefixes: ``module.``, ``_orig_mod.``, ``_fsdp_wrapped_module.``, ``base_model.model.``."""
    out = {}
    for k, v in state_dict.items():
        changed = True
        while changed:
            changed = False
            for pre in ("module.", "_orig_mod.", "_fsdp_wrapped_module.", "base_model.model."):
                if k.startswith(pre):
                    k, changed = k[len(pre):], True
        out[k.replace("._fsdp_wrapped_module", "").replace("._orig_mod", "")] = v
    return out


def extract_multi_modal_inputs(batch_data: list[dict], indices=None) -> dict:
    """Concatenate the per-sample ``multi_modal_inputs`` dicts of a batch key by key (verl/utils/model.py:696-738);
    ``indices`` selects samples."""
    picked = batch_data if indices is None else [batch_data[int(i)] for i in indices]
    keys = sorted({k for d in picked if d for k in d})
    out = {}
    for k in keys:
        vals = [d[k] for d in picked if d and k in d]
        out[k] = torch.cat(vals, dim=0) if all(isinstance(v, torch.Tensor) for v in vals) else vals
    return out


def check_exclude_modules(config, key: str) -> bool:
    """True when the module named ``key`` is excluded by an adapter config's ``exclude_modules`` (a regular expression
    given as a string, or a list of module names / name suffixes)."""
    excl = getattr(config, "exclude_modules", None) if not isinstance(config, dict) else config.get("exclude_modules")
    if not excl:
        return False
    if isinstance(excl, str):
        import re

        return re.fullmatch(excl, key) is not None
    return key in excl or any(key.endswith(f".{e}") for e in excl)


def get_generation_config(model: str, trust_remote_code: bool = False):
    """``generation_config.json`` of a checkpoint directory (or the defaults derived from its ``config.json``); None when
    neither is there."""
    try:
        from transformers import AutoConfig, GenerationConfig
    except ImportError:
        return None
    try:
        return GenerationConfig.from_pretrained(model)
    except (OSError, ValueError):
        try:
            return GenerationConfig.from_model_config(AutoConfig.from_pretrained(model, trust_remote_code=trust_remote_code))
        except (OSError, ValueError):
            return None


def get_hf_model_path(config) -> str:
    """Local directory of ``config.model.path`` (remote paths are fetched first)."""
    from .fs import copy_to_local, is_non_local

    path = config.model.path
    return copy_to_local(path, use_shm=bool(config.model.get("use_shm", False))) if is_non_local(path) else path


class LambdaLayer(nn.Module):
    def __init__(self, fn):
        super().__init__()
        self.fn = fn

    def forward(self, *args, **kwargs):
        return self.fn(*args, **kwargs)


def squeeze(x: torch.Tensor) -> torch.Tensor:
    return torch.squeeze(x, dim=-1)
