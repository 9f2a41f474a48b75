"""Dependency-free configuration system: YAML composition with ``defaults:`` lists,
``${...}`` / ``${oc.select:key,default}`` interpolation, the Hydra override grammar
(``a.b=v``, ``+a.b=v``, ``++a.b=v``, ``~a.b``) and ``_target_`` instantiation into dataclasses.

The reference uses Hydra + OmegaConf for this (verl/trainer/main_ppo.py:35-45,
verl/utils/config.py:23-66 ``omega_conf_to_dataclass``, :74-213 ``validate_config``); neither is
a dependency here.
"""

from __future__ import annotations

import copy
import importlib
import re
from dataclasses import fields, is_dataclass
from pathlib import Path
from typing import Any, Iterable, Optional

import yaml

MISSING = "???"


class _Loader(yaml.SafeLoader):
    """SafeLoader that also reads ``1e-6`` (no dot) as a float, as OmegaConf does."""


_Loader.add_implicit_resolver(
    "tag:yaml.org,2002:float",
    re.compile(r"""^(?:[-+]?(?:[0-9][0-9_]*)\.[0-9_]*(?:[eE][-+]?[0-9]+)?
                   |[-+]?(?:[0-9][0-9_]*)(?:[eE][-+]?[0-9]+)
                   |\.[0-9_]+(?:[eE][-+]?[0-9]+)?
                   |[-+]?\.(?:inf|Inf|INF)
                   |\.(?:nan|NaN|NAN))$""", re.X),
    list("-+0123456789."))


def _yaml_load(text):
    return yaml.load(text, Loader=_Loader)


class ConfigDict(dict):
    """Nested dict with attribute access (the role of OmegaConf's DictConfig)."""

    def __getattr__(self, key):
        try:
            return self[key]
        except KeyError as e:
            raise AttributeError(key) from e

    def __setattr__(self, key, value):
        self[key] = value

    def __delattr__(self, key):
        try:
            del self[key]
        except KeyError as e:
            raise AttributeError(key) from e

    def __deepcopy__(self, memo):
        return ConfigDict({k: copy.deepcopy(v, memo) for k, v in self.items()})

    def to_container(self) -> dict:
        return to_container(self)


def to_config(obj):
    if isinstance(obj, dict):
        return ConfigDict({k: to_config(v) for k, v in obj.items()})
    if isinstance(obj, (list, tuple)):
        return [to_config(v) for v in obj]
    return obj


def to_container(obj):
    if isinstance(obj, dict):
        return {k: to_container(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [to_container(v) for v in obj]
    return obj


# --------------------------------------------------------------------- path helpers
def select(cfg, path: str, default=None):
    cur = cfg
    for part in path.split("."):
        if isinstance(cur, dict) and part in cur:
            cur = cur[part]
        elif isinstance(cur, list) and part.isdigit() and int(part) < len(cur):
            cur = cur[int(part)]
        else:
            return default
    return cur


def set_path(cfg: dict, path: str, value, create: bool = True) -> None:
    parts = path.split(".")
    cur = cfg
    for p in parts[:-1]:
        if p not in cur or not isinstance(cur[p], dict):
            if not create:
                raise KeyError(f"config path '{path}' does not exist (use +{path}=... to add it)")
            cur[p] = ConfigDict()
        cur = cur[p]
    cur[parts[-1]] = value


def del_path(cfg: dict, path: str) -> None:
    parts = path.split(".")
    cur = cfg
    for p in parts[:-1]:
        cur = cur[p]
    del cur[parts[-1]]


def merge(base: dict, other: dict) -> dict:
    """Recursive in-place merge of ``other`` into ``base`` (lists and scalars replace)."""
    for k, v in other.items():
        if isinstance(v, dict) and isinstance(base.get(k), dict):
            merge(base[k], v)
        else:
            base[k] = copy.deepcopy(v)
    return base


# ----------------------------------------------------------------------- overrides
def _parse_value(text: str):
    text = text.strip()
    if text == "":
        return ""
    try:
        return _yaml_load(text)
    except yaml.YAMLError:
        return text


_OVERRIDE = re.compile(r"^(?P<prefix>\+\+|\+|~)?(?P<key>[^=]+?)(=(?P<value>.*))?$", re.S)


def apply_overrides(cfg: dict, overrides: Iterable[str]) -> dict:
    for ov in overrides:
        m = _OVERRIDE.match(ov.strip())
        if not m:
            raise ValueError(f"cannot parse override '{ov}'")
        prefix, key, value = m.group("prefix") or "", m.group("key").strip(), m.group("value")
        if prefix == "~":
            del_path(cfg, key)
            continue
        if value is None:
            raise ValueError(f"override '{ov}' needs a value")
        val = to_config(_parse_value(value))
        if prefix == "":
            if select(cfg, key, default=_SENTINEL) is _SENTINEL:
                raise KeyError(f"Could not override '{key}': key not in config (use +{key}={value} to append)")
            set_path(cfg, key, val, create=False)
        else:
            set_path(cfg, key, val, create=True)
    return cfg


_SENTINEL = object()

# ------------------------------------------------------------------- interpolation
_INTERP = re.compile(r"\$\{([^${}]+)\}")


def _resolve_ref(expr: str, root, here_path: list[str]):
    expr = expr.strip()
    if expr.startswith("oc.select:"):
        body = expr[len("oc.select:"):]
        key, _, default = body.partition(",")
        got = _lookup(key.strip(), root, here_path)
        if got is _SENTINEL or got is None:
            return _parse_value(default) if default != "" else None
        return got
    if expr.startswith("oc.env:"):
        import os

        key, _, default = expr[len("oc.env:"):].partition(",")
        return os.environ.get(key.strip(), _parse_value(default) if default else None)
    got = _lookup(expr, root, here_path)
    if got is _SENTINEL:
        raise KeyError(f"interpolation key '{expr}' not found")
    return got


def _lookup(key: str, root, here_path: list[str]):
    if key.startswith("."):
        up = len(key) - len(key.lstrip("."))
        base = here_path[: len(here_path) - (up - 1)]  # one dot = the node that holds this value
        key = ".".join(base + [key.lstrip(".")]) if key.lstrip(".") else ".".join(base)
    return select(root, key, default=_SENTINEL)


def _resolve_value(val, root, here_path, depth=0):
    if depth > 20:
        raise RecursionError("interpolation too deep")
    if not isinstance(val, str) or "${" not in val:
        return val
    whole = _INTERP.fullmatch(val.strip())
    if whole:
        res = _resolve_ref(whole.group(1), root, here_path)
        if isinstance(res, str):
            return _resolve_value(res, root, here_path, depth + 1)
        return copy.deepcopy(res)
    out = val
    while True:
        m = _INTERP.search(out)
        if not m:
            return out
        res = _resolve_value(_resolve_ref(m.group(1), root, here_path), root, here_path, depth + 1)
        out = out[: m.start()] + str(res) + out[m.end():]


def resolve(cfg, root=None, path: Optional[list[str]] = None):
    """Resolve all interpolations in place (relative keys ``${.x}`` / ``${..x}`` are relative to the node)."""
    root = cfg if root is None else root
    path = path or []
    if isinstance(cfg, dict):
        for k in list(cfg.keys()):
            v = cfg[k]
            if isinstance(v, (dict, list)):
                resolve(v, root, path + [k])
            else:
                cfg[k] = _resolve_value(v, root, path)
        # a second pass lets values that referenced still-unresolved nodes settle
        for k in list(cfg.keys()):
            if isinstance(cfg[k], str) and "${" in cfg[k]:
                cfg[k] = _resolve_value(cfg[k], root, path)
    elif isinstance(cfg, list):
        for i, v in enumerate(cfg):
            if isinstance(v, (dict, list)):
                resolve(v, root, path + [str(i)])
            else:
                cfg[i] = _resolve_value(v, root, path)
    return cfg


# --------------------------------------------------------------------- composition
def _load_yaml(path: Path) -> dict:
    with open(path) as f:
        return _yaml_load(f) or {}


def _find(config_dir: Path, name: str) -> Path:
    for ext in (".yaml", ".yml", ""):
        p = config_dir / (name + ext)
        if p.is_file():
            return p
    raise FileNotFoundError(f"config '{name}' not found under {config_dir}")


def _compose_file(config_dir: Path, name: str, group_choice: dict[str, str]) -> dict:
    raw = _load_yaml(_find(config_dir, name))
    defaults = raw.pop("defaults", None)
    if not defaults:
        return raw
    out: dict = {}
    self_done = False
    parent_group = str(Path(name).parent) if "/" in name else ""
    for item in defaults:
        if item == "_self_":
            merge(out, raw)
            self_done = True
            continue
        if isinstance(item, str):
            fname, _, package = item.partition("@")
            sub_name = f"{parent_group}/{fname}" if parent_group and not fname.startswith("/") else fname.lstrip("/")
            sub = _compose_file(config_dir, sub_name, group_choice)
            if package:
                node = ConfigDict()
                set_path(node, package, sub)
                sub = node
            merge(out, sub)
            continue
        (k, v), = item.items()
        if v is None:
            continue
        optional = k.startswith("optional ")
        k = k.replace("optional ", "").replace("override ", "").strip()
        group, _, package = k.partition("@")
        group = group.lstrip("/")
        choice = group_choice.get(group, v)
        try:
            sub = _compose_file(config_dir, f"{group}/{choice}", group_choice)
        except FileNotFoundError:
            if optional:
                continue
            raise
        package = package or group.replace("/", ".")
        if package == "_global_":
            merge(out, sub)
        else:
            node = ConfigDict()
            set_path(node, package, sub)
            merge(out, node)
    if not self_done:
        merge(out, raw)
    return out


# engine keys of the reference's Megatron strategy that name something the one native engine has
_MEGATRON_ENGINE_KEYS = {"tensor_model_parallel_size", "pipeline_model_parallel_size", "expert_model_parallel_size",
                         "context_parallel_size", "param_offload", "optimizer_offload", "grad_offload", "seed", "forward_only",
                         "full_determinism"}
_MEGATRON_LR_STYLE = {"constant": "constant", "cosine": "cosine", "WSD": "wsd", "wsd": "wsd"}


def translate_megatron_overrides(overrides: Iterable[str]) -> tuple[list[str], list[str]]:
    """Command lines written for the reference's Megatron strategy (``--config-name ppo_megatron_trainer``,
    ``<role>.strategy=megatron``, ``<role>.megatron.tensor_model_parallel_size=2`` ...,
    verl/trainer/config/ppo_megatron_trainer.yaml) onto this framework's one engine: the parallel sizes, offload switches
    and the seed go to ``<role>.fsdp_config`` (``critic.model.fsdp_config`` for the critic), the strategy becomes the
    native one, ``optim.lr_decay_style`` becomes ``optim.lr_scheduler_type``. Keys that configure Megatron-core itself
    (transformer overrides, distributed optimizer, dist checkpointing, mbridge) have no counterpart: they are returned
    in the second list and left out. Virtual pipeline stages are refused."""
    out, dropped = [], []
    for ov in overrides:
        m = _OVERRIDE.match(ov)
        key = m.group("key").strip() if m else ""
        val = m.group("value") if m else None
        pre = (m.group("prefix") or "") if m else ""
        if key.endswith(".strategy") and val == "megatron":
            out.append(f"{pre}{key}=fsdp")
            continue
        if ".megatron." in key:
            role, leaf = key.split(".megatron.", 1)
            if leaf == "virtual_pipeline_model_parallel_size" and val not in (None, "null", "None", "1"):
                raise NotImplementedError("virtual pipeline stages (virtual_pipeline_model_parallel_size) are not supported")
            if leaf in _MEGATRON_ENGINE_KEYS:
                home = f"{role}.model.fsdp_config" if role == "critic" else f"{role}.fsdp_config"
                out.append(f"{home}.{leaf}={val}")
            else:
                dropped.append(ov)
            continue
        if key.endswith(".optim.lr_decay_style") or key == "optim.lr_decay_style":
            if val not in _MEGATRON_LR_STYLE:
                raise NotImplementedError(f"optim.lr_decay_style={val}: supported are {sorted(set(_MEGATRON_LR_STYLE))}")
            out.append(f"{pre}{key[: -len('lr_decay_style')]}lr_scheduler_type={_MEGATRON_LR_STYLE[val]}")
            continue
        if key.endswith((".optim.use_checkpoint_opt_param_scheduler", ".optim.lr_warmup_init", ".optim.lr_decay_steps",
                         ".optim.weight_decay_incr_style", ".optim.lr_wsd_decay_style", ".optim.lr_wsd_decay_steps",
                         ".optim.min_lr", ".load_weight")):
            dropped.append(ov)
            continue
        out.append(ov)
    return out, dropped


def compose(config_name: str, overrides: Optional[Iterable[str]] = None, config_dir: str | Path | None = None,
            resolve_interpolations: bool = True) -> ConfigDict:
    """Load ``config_name`` (with its ``defaults:`` tree) from ``config_dir``, apply CLI-style overrides."""
    if config_dir is None:
        config_dir = Path(__file__).resolve().parent.parent / "trainer" / "config"
    config_dir = Path(config_dir)
    overrides = list(overrides or [])
    if config_name == "ppo_megatron_trainer" or any(".megatron." in o or o.endswith("strategy=megatron") or
                                                    "lr_decay_style=" in o for o in overrides):
        overrides, dropped = translate_megatron_overrides(overrides)
        if config_name == "ppo_megatron_trainer":
            config_name = "ppo_trainer"
        if dropped:
            print(f"[config] Megatron-core options without a counterpart here were left out: {dropped}")
    group_choice, value_overrides = {}, []
    for ov in overrides:
        m = _OVERRIDE.match(ov)
        key = m.group("key").strip() if m else ""
        val = m.group("value") if m else None
        # "group=choice" selects a defaults-list option when group is a directory of configs
        if m and not m.group("prefix") and val is not None and (config_dir / key.split("@")[0]).is_dir() \
                and "." not in key and _is_choice(config_dir / key.split("@")[0], val):
            group_choice[key.split("@")[0]] = val
        else:
            value_overrides.append(ov)
    cfg = to_config(_compose_file(config_dir, config_name, group_choice))
    apply_overrides(cfg, value_overrides)
    if resolve_interpolations:
        resolve(cfg)
    return cfg


def compose_from_dict(defaults: dict, overrides: Optional[Iterable[str]] = None, resolve_interpolations: bool = True) -> ConfigDict:
    """Config for small entry points that ship their defaults as a dict: copy, apply ``a.b=c`` overrides, resolve."""
    import copy

    cfg = apply_overrides(copy.deepcopy(defaults), list(overrides or []))
    cfg = to_config(cfg)
    return resolve(cfg) if resolve_interpolations else cfg


def _is_choice(group_dir: Path, val: str) -> bool:
    return any((group_dir / (val + ext)).is_file() for ext in (".yaml", ".yml"))


# ------------------------------------------------------------------ dataclass bridge
def _locate(target: str):
    mod, _, name = target.rpartition(".")
    # accept the reference's module paths for the same class names
    if mod.startswith("verl.") or mod == "verl":
        mod = "verl_b200" + mod[len("verl"):]
    return getattr(importlib.import_module(mod), name)


def omega_conf_to_dataclass(config, dataclass_type=None):
    """Instantiate the dataclass named by ``_target_`` (or ``dataclass_type``) from a config node,
    recursing into nested nodes that carry their own ``_target_``."""
    if config is None:
        return dataclass_type() if dataclass_type is not None and is_dataclass(dataclass_type) else None
    if is_dataclass(config) and not isinstance(config, type):
        return config
    if not isinstance(config, dict):
        return config
    target = config.get("_target_")
    cls = dataclass_type or (_locate(target) if target else None)
    if cls is None:
        return config
    names = {f.name for f in fields(cls)}
    kwargs = {}
    for k, v in config.items():
        if k == "_target_":
            if "_target_" in names:
                kwargs[k] = v
            continue
        if k not in names:
            raise TypeError(f"{cls.__name__} got an unexpected config key '{k}'")
        if isinstance(v, dict) and v.get("_target_"):
            v = omega_conf_to_dataclass(v)
        kwargs[k] = v
    return cls(**kwargs)


def update_dict_with_config(dictionary: dict, config) -> None:
    for key in dictionary:
        if hasattr(config, key):
            dictionary[key] = getattr(config, key)


# ---------------------------------------------------------------------- validation
def validate_config(config, use_reference_policy: bool, use_critic: bool) -> None:
    """Cross-field checks before a PPO run (batch divisibility, exclusive micro-batch options,
    sampling sanity). Mirrors the checks of verl/utils/config.py:74-213."""
    tr = config.trainer
    n_gpus = tr.n_gpus_per_node * tr.nnodes
    ar = config.actor_rollout_ref
    if not ar.actor.get("use_dynamic_bsz", False):
        real_bsz = config.data.train_batch_size * ar.rollout.n
        assert real_bsz % n_gpus == 0, (
            f"real_train_batch_size ({real_bsz}) must be divisible by total n_gpus ({n_gpus}).")

    def exclusive(mbs, mbs_per_gpu, name):
        param, per_gpu = "micro_batch_size", "micro_batch_size_per_gpu"
        if mbs is None and mbs_per_gpu is None:
            raise ValueError(f"[{name}] Please set at least one of '{name}.{param}' or '{name}.{per_gpu}'.")
        if mbs is not None and mbs_per_gpu is not None:
            raise ValueError(f"[{name}] You have set both '{name}.{param}' AND '{name}.{per_gpu}'. Please remove "
                             f"'{name}.{param}' because only '*_{per_gpu}' is supported (the former is deprecated).")

    if not ar.actor.get("use_dynamic_bsz", False):
        if use_reference_policy:
            exclusive(ar.ref.get("log_prob_micro_batch_size"), ar.ref.get("log_prob_micro_batch_size_per_gpu"),
                      "actor_rollout_ref.ref.log_prob")
        exclusive(ar.rollout.get("log_prob_micro_batch_size"), ar.rollout.get("log_prob_micro_batch_size_per_gpu"),
                  "actor_rollout_ref.rollout.log_prob")
        exclusive(ar.actor.get("ppo_micro_batch_size"), ar.actor.get("ppo_micro_batch_size_per_gpu"),
                  "actor_rollout_ref.actor.ppo")
        mini = ar.actor.ppo_mini_batch_size
        assert config.data.train_batch_size >= mini, (
            f"train_batch_size ({config.data.train_batch_size}) must be >= ppo_mini_batch_size ({mini})")
    if use_critic and not config.critic.get("use_dynamic_bsz", False):
        exclusive(config.critic.get("ppo_micro_batch_size"), config.critic.get("ppo_micro_batch_size_per_gpu"), "critic.ppo")
    if config.algorithm.get("use_kl_in_reward", False) and ar.actor.get("use_kl_loss", False):
        print("NOTICE: You have both enabled in-reward kl and kl loss.")
    val = ar.rollout.get("val_kwargs", {}) or {}
    if val.get("do_sample", False):
        assert ar.rollout.temperature > 0, "validation gen temperature should be greater than 0 when enabling do_sample"
    lora_rank = ar.model.get("lora_rank", 0) or 0
    assert lora_rank >= 0, "lora_rank must be non-negative"
    print("[validate_config] All configuration checks passed successfully!")
