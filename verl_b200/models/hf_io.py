"""HuggingFace checkpoint compatibility: parameter-name mapping between the HF layout
(separate q/k/v and gate/up projections, per-expert MoE tensors) and this framework's fused
layout, plus safetensors import/export.

The reference loads/saves HF models directly through ``transformers``
(verl/utils/checkpoint/fsdp_checkpoint_manager.py:303-348) and regroups fused tensors for
inference engines in verl/utils/megatron_utils.py:846 (default_tp_concat_fn).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Iterable, Iterator

import torch

from .config import ModelConfig


_VIS_HF_TO_NATIVE = (("attn.qkv.", "qkv."), ("attn.proj.", "proj."), ("mlp.fc1.", "fc1."), ("mlp.fc2.", "fc2."),
                     ("mlp.gate_proj.", "fc_gate."), ("mlp.up_proj.", "fc_up."), ("mlp.down_proj.", "fc2."),
                     ("merger.ln_q.", "ln_q."), ("merger.mlp.0.", "merge_fc1."), ("merger.mlp.2.", "merge_fc2."),
                     ("patch_embed.proj.", "patch_embed."))


# Qwen3-VL names its MLP and merger linears differently and adds a position table and the deepstack mergers
_VIS3_HF_TO_NATIVE = (("attn.qkv.", "qkv."), ("attn.proj.", "proj."), ("mlp.linear_fc1.", "fc1."), ("mlp.linear_fc2.", "fc2."),
                      ("visual.merger.norm.", "visual.ln_q."), ("visual.merger.linear_fc1.", "visual.merge_fc1."),
                      ("visual.merger.linear_fc2.", "visual.merge_fc2."), ("deepstack_merger_list.", "deepstack."),
                      ("patch_embed.proj.", "patch_embed."))


def _vis3_hf_to_native(name: str) -> str:
    for a, b in _VIS3_HF_TO_NATIVE:
        name = name.replace(a, b)
    if name.startswith("visual.deepstack."):
        name = name.replace(".linear_fc1.", ".fc1.").replace(".linear_fc2.", ".fc2.")
    return name


def _vis3_native_to_hf(name: str) -> str:
    if name.startswith("visual.deepstack."):
        return name.replace("visual.deepstack.", "visual.deepstack_merger_list.").replace(".fc1.", ".linear_fc1.").replace(
            ".fc2.", ".linear_fc2.")
    for hf, nat in (("visual.merger.norm.", "visual.ln_q."), ("visual.merger.linear_fc1.", "visual.merge_fc1."),
                    ("visual.merger.linear_fc2.", "visual.merge_fc2."), ("visual.patch_embed.proj.", "visual.patch_embed.")):
        if name.startswith(nat):
            return hf + name[len(nat):]
    if name.startswith("visual.blocks."):
        for hf, nat in ((".attn.qkv.", ".qkv."), (".attn.proj.", ".proj."), (".mlp.linear_fc1.", ".fc1."),
                        (".mlp.linear_fc2.", ".fc2.")):
            if nat in name:
                return name.replace(nat, hf)
    return name


def _normalise_vl_keys(hf_sd: dict) -> dict:
    """Vision-language checkpoints: ``model.language_model.*`` (recent HF) or ``model.*`` (original release) for the
    decoder, ``model.visual.*`` or ``visual.*`` for the tower -> ``model.*`` and ``visual.*``."""
    out = {}
    for k, v in hf_sd.items():
        if k.startswith("model.language_model."):
            k = "model." + k[len("model.language_model."):]
        elif k.startswith("model.visual."):
            k = k[len("model."):]
        out[k] = v
    return out


def hf_to_native_state_dict(cfg: ModelConfig, hf_sd: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """Fuse an HF state dict into native parameter names/shapes."""
    out: dict[str, torch.Tensor] = {}
    if cfg.is_vl or any(k.startswith(("model.language_model.", "model.visual.", "visual.")) for k in hf_sd):
        hf_sd = _normalise_vl_keys(hf_sd)
        for k, v in hf_sd.items():
            if not k.startswith("visual."):
                continue
            n = k
            if cfg.model_type in ("qwen3_vl", "qwen3_vl_moe"):
                n = _vis3_hf_to_native(n)
            else:
                for a, b in _VIS_HF_TO_NATIVE:
                    n = n.replace(a, b)
            out[n] = v.reshape(v.shape[0], -1) if n == "visual.patch_embed.weight" else v
    g = lambda k: hf_sd[k]  # noqa: E731
    out["embed_tokens.weight"] = g("model.embed_tokens.weight")
    out["norm.weight"] = g("model.norm.weight")
    if "lm_head.weight" in hf_sd and not cfg.tie_word_embeddings:
        out["lm_head.weight"] = g("lm_head.weight")
    if "score.weight" in hf_sd:
        out["score.weight"] = g("score.weight")
    apertus = cfg.model_type == "apertus"  # other names for the two norms, a two-matrix MLP with activation parameters
    for i in range(cfg.num_hidden_layers):
        p, n = f"model.layers.{i}.", f"layers.{i}."
        out[n + "input_layernorm.weight"] = g(p + ("attention_layernorm.weight" if apertus else "input_layernorm.weight"))
        out[n + "post_attention_layernorm.weight"] = g(p + ("feedforward_layernorm.weight" if apertus else
                                                           "post_attention_layernorm.weight"))
        out[n + "self_attn.qkv_proj.weight"] = torch.cat(
            [g(p + f"self_attn.{x}_proj.weight") for x in "qkv"], dim=0)
        if cfg.attention_bias:
            out[n + "self_attn.qkv_proj.bias"] = torch.cat([g(p + f"self_attn.{x}_proj.bias") for x in "qkv"], dim=0)
        out[n + "self_attn.o_proj.weight"] = g(p + "self_attn.o_proj.weight")
        if cfg.qk_norm:
            out[n + "self_attn.q_norm.weight"] = g(p + "self_attn.q_norm.weight")
            out[n + "self_attn.k_norm.weight"] = g(p + "self_attn.k_norm.weight")
        if cfg.is_moe and (p + "mlp.experts.gate_up_proj") in hf_sd:
            # experts stored as stacked tensors [E, 2I, H] / [E, H, I] (Qwen3-VL-MoE): the native layout
            out[n + "mlp.gate.weight"] = g(p + "mlp.gate.weight")
            out[n + "mlp.gate_up_proj"] = g(p + "mlp.experts.gate_up_proj")
            out[n + "mlp.down_proj"] = g(p + "mlp.experts.down_proj")
        elif cfg.is_moe:
            out[n + "mlp.gate.weight"] = g(p + "mlp.gate.weight")
            out[n + "mlp.gate_up_proj"] = torch.stack([
                torch.cat([g(p + f"mlp.experts.{e}.gate_proj.weight"), g(p + f"mlp.experts.{e}.up_proj.weight")], 0)
                for e in range(cfg.num_experts)])
            out[n + "mlp.down_proj"] = torch.stack(
                [g(p + f"mlp.experts.{e}.down_proj.weight") for e in range(cfg.num_experts)])
        elif not cfg.mlp_gated:
            out[n + "mlp.up_proj.weight"] = g(p + "mlp.up_proj.weight")
            out[n + "mlp.down_proj.weight"] = g(p + "mlp.down_proj.weight")
            out[n + "mlp.act_alpha_p"] = g(p + "mlp.act_fn.alpha_p").reshape(1)
            out[n + "mlp.act_alpha_n"] = g(p + "mlp.act_fn.alpha_n").reshape(1)
        else:
            out[n + "mlp.gate_up_proj.weight"] = torch.cat(
                [g(p + "mlp.gate_proj.weight"), g(p + "mlp.up_proj.weight")], dim=0)
            out[n + "mlp.down_proj.weight"] = g(p + "mlp.down_proj.weight")
    return out


def native_to_hf_items(cfg: ModelConfig, named: Iterable[tuple[str, torch.Tensor]]) -> Iterator[tuple[str, torch.Tensor]]:
    """Stream (hf_name, tensor) pairs from native (name, tensor) pairs, splitting fused tensors.
    Works one parameter at a time so it can drive a weight-sync generator."""
    vl = cfg.is_vl
    lm = "model.language_model." if vl else "model."
    for name, t in named:
        if name.startswith("visual.") and cfg.model_type in ("qwen3_vl", "qwen3_vl_moe"):
            if name == "visual.patch_embed.weight":
                vc = cfg.extra["vision_config"]
                t = t.reshape(t.shape[0], vc.get("in_channels", 3), vc.get("temporal_patch_size", 2), vc.get("patch_size", 16),
                              vc.get("patch_size", 16))
            yield "model." + _vis3_native_to_hf(name), t
            continue
        if name.startswith("visual."):
            n = _vis_native_to_hf(name, gated=(cfg.extra.get("vision_config") or {}).get("intermediate_size") is not None
                                  or cfg.model_type == "qwen2_5_vl")
            if name == "visual.patch_embed.weight":
                vc = cfg.extra["vision_config"]
                t = t.reshape(t.shape[0], vc.get("in_channels", 3), vc.get("temporal_patch_size", 2), vc.get("patch_size", 14),
                              vc.get("patch_size", 14))
            yield "model." + n, t
            continue
        if vl and name in ("embed_tokens.weight", "norm.weight"):
            yield lm + name, t
            continue
        if vl and name.startswith("layers."):
            for hn, ht in native_to_hf_items(_text_only(cfg), [(name, t)]):
                yield lm + hn[len("model."):], ht
            continue
        if name == "embed_tokens.weight":
            yield "model.embed_tokens.weight", t
        elif name == "norm.weight":
            yield "model.norm.weight", t
        elif name in ("lm_head.weight", "score.weight"):
            yield name, t
        elif name.startswith("layers."):
            _, idx, rest = name.split(".", 2)
            p = f"model.layers.{idx}."
            if rest == "self_attn.qkv_proj.weight" or rest == "self_attn.qkv_proj.bias":
                kind = rest.rsplit(".", 1)[1]
                q, k, v = t.split([cfg.q_size, cfg.kv_size, cfg.kv_size], dim=0)
                yield p + f"self_attn.q_proj.{kind}", q
                yield p + f"self_attn.k_proj.{kind}", k
                yield p + f"self_attn.v_proj.{kind}", v
            elif cfg.model_type == "apertus" and rest in ("input_layernorm.weight", "post_attention_layernorm.weight"):
                yield p + ("attention_layernorm.weight" if rest.startswith("input") else "feedforward_layernorm.weight"), t
            elif rest in ("mlp.act_alpha_p", "mlp.act_alpha_n"):
                yield p + "mlp.act_fn." + rest[len("mlp.act_"):], t
                if rest.endswith("_n"):  # the two constants of the activation are buffers of the HF module
                    yield p + "mlp.act_fn.beta", torch.tensor(0.5, dtype=t.dtype)
                    yield p + "mlp.act_fn.eps", torch.tensor(-1e-6, dtype=t.dtype)
            elif rest == "mlp.gate_up_proj.weight":
                gte, up = t.chunk(2, dim=0)
                yield p + "mlp.gate_proj.weight", gte
                yield p + "mlp.up_proj.weight", up
            elif rest in ("mlp.gate_up_proj", "mlp.down_proj") and cfg.model_type == "qwen3_vl_moe":
                yield p + "mlp.experts." + rest[len("mlp."):], t
            elif rest == "mlp.gate_up_proj":
                for e in range(t.shape[0]):
                    gte, up = t[e].chunk(2, dim=0)
                    yield p + f"mlp.experts.{e}.gate_proj.weight", gte
                    yield p + f"mlp.experts.{e}.up_proj.weight", up
            elif rest == "mlp.down_proj":
                for e in range(t.shape[0]):
                    yield p + f"mlp.experts.{e}.down_proj.weight", t[e]
            else:
                yield p + rest, t
        else:
            yield name, t


def _vis_native_to_hf(name: str, gated: bool = False) -> str:
    """``gated``: the Qwen2.5-VL tower (gate / up / down projections) rather than the Qwen2-VL one (fc1 / fc2)."""
    body = name[len("visual."):]
    parts = body.split(".")
    # blocks.N.<x>.<w|b> or top-level <x>.<w|b>
    leaf = parts[-2] + "."
    for hf, nat in _VIS_HF_TO_NATIVE:
        if leaf == nat:
            if nat == "fc2." and gated != (hf == "mlp.down_proj."):
                continue
            return "visual." + ".".join(parts[:-2] + [hf[:-1], parts[-1]])
    return name


def _text_only(cfg: ModelConfig) -> ModelConfig:
    import dataclasses

    return dataclasses.replace(cfg, extra={})


def native_to_hf_state_dict(cfg: ModelConfig, sd: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    return {k: v for k, v in native_to_hf_items(cfg, sd.items())}


def save_hf_checkpoint(cfg: ModelConfig, native_sd: dict[str, torch.Tensor], path: str | Path,
                       dtype: torch.dtype = torch.bfloat16, max_shard_bytes: int = 5 * 1024**3) -> None:
    """Write ``config.json`` + sharded ``model-xxxxx-of-xxxxx.safetensors`` (+ index) in HF layout."""
    from safetensors.torch import save_file

    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    cfg.save_pretrained(path)
    shards, cur, cur_bytes = [], {}, 0
    for k, v in native_to_hf_items(cfg, native_sd.items()):
        t = v.detach().to(dtype).cpu().contiguous()
        nbytes = t.numel() * t.element_size()
        if cur and cur_bytes + nbytes > max_shard_bytes:
            shards.append(cur)
            cur, cur_bytes = {}, 0
        cur[k] = t
        cur_bytes += nbytes
    if cur:
        shards.append(cur)
    if len(shards) == 1:
        save_file(shards[0], str(path / "model.safetensors"), metadata={"format": "pt"})
        return
    index = {"metadata": {"total_size": 0}, "weight_map": {}}
    for i, sh in enumerate(shards):
        fname = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, str(path / fname), metadata={"format": "pt"})
        for k, t in sh.items():
            index["weight_map"][k] = fname
            index["metadata"]["total_size"] += t.numel() * t.element_size()
    (path / "model.safetensors.index.json").write_text(json.dumps(index, indent=2))


def load_hf_checkpoint(path: str | Path) -> tuple[ModelConfig, dict[str, torch.Tensor]]:
    """Read an HF directory (safetensors, single or sharded) into a native state dict."""
    from safetensors.torch import load_file

    path = Path(path)
    cfg = ModelConfig.from_pretrained(path)
    hf_sd: dict[str, torch.Tensor] = {}
    files = sorted(path.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors files under {path}")
    for f in files:
        hf_sd.update(load_file(str(f)))
    return cfg, hf_to_native_state_dict(cfg, hf_sd)
