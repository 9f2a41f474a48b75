"""Build interactions from YAML (verl/interactions/utils/interaction_registry.py): ``interaction: [{name, class_name, config}]``."""

from __future__ import annotations

import importlib

import yaml


def get_interaction_class(cls_name: str):
    mod, name = cls_name.rsplit(".", 1)
    if mod.startswith("verl."):
        mod = "verl_b200." + mod[len("verl."):]
    return getattr(importlib.import_module(mod), name)


def initialize_interactions_from_config(interaction_config_file: str) -> dict:
    with open(interaction_config_file) as f:
        conf = yaml.safe_load(f) or {}
    out = {}
    for ic in conf.get("interaction", []):
        cls = get_interaction_class(ic["class_name"])
        name = ic.get("name") or cls.__name__.replace("Interaction", "").lower()
        if name in out:
            raise ValueError(f"Duplicate interaction name '{name}' found. Each interaction must have a unique name.")
        cfg = dict(ic.get("config") or {})
        cfg["name"] = name
        out[name] = cls(config=cfg)
    return out
