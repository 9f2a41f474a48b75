"""Entry point: ``python -m verl_b200.trainer.main_ppo key=value ...`` (Hydra-style overrides).

Mirrors verl/trainer/main_ppo.py:35-448: compose ``ppo_trainer.yaml`` + overrides, map roles to worker
classes and resource pools, build tokenizer / datasets / reward functions, run ``RayPPOTrainer.fit()``.
Launched under ``torchrun`` (WORLD_SIZE set) it runs in SPMD mode: one controller replica per GPU.
"""

from __future__ import annotations

import os
import sys
from typing import Optional

from ..utils.config import compose, validate_config
from .ppo.utils import Role, need_critic, need_reference_policy


def create_rl_dataset(data_paths, data_config, tokenizer, processor=None, is_train=True, max_samples: int = -1):
    """``data.custom_cls`` (path + name), a ``synthetic:`` spec, or the parquet/json RLHFDataset."""
    from ..utils.dataset import RLHFDataset, SyntheticPromptDataset
    from ..utils.py_functional import load_extern_object

    cc = data_config.get("custom_cls") or {}
    if cc.get("path"):
        cls = load_extern_object(cc["path"], cc["name"])
        return cls(data_files=data_paths, tokenizer=tokenizer, processor=processor, config=data_config)
    if isinstance(data_paths, str) and data_paths.startswith("synthetic:"):
        # synthetic:<num>:<min_len>:<max_len>:<id_lo>:<id_hi>:<seed>[:<data_source>[:<ground_truth>]]
        parts = data_paths.split(":")
        num, lo, hi, id_lo, id_hi, seed = (int(x) for x in parts[1:7])
        source = parts[7] if len(parts) > 7 else "synthetic/even_fraction"
        gt = int(parts[8]) if len(parts) > 8 else None
        return SyntheticPromptDataset(num, lo, hi, id_lo, id_hi, data_config.max_prompt_length, seed, source,
                                      getattr(tokenizer, "pad_token_id", 0) or 0, gt)
    return RLHFDataset(data_paths, tokenizer, data_config, processor, max_samples)


def create_rl_sampler(data_config, dataset):
    import torch
    from torch.utils.data import RandomSampler, SequentialSampler

    sc = data_config.get("sampler") or {}
    if sc.get("class_path"):
        from ..utils.py_functional import load_extern_object

        return load_extern_object(sc["class_path"], sc["class_name"])(data_source=dataset, data_config=data_config)
    if data_config.get("shuffle", True):
        g = torch.Generator()
        g.manual_seed(int(data_config.get("seed") or 1))
        return RandomSampler(dataset, generator=g)
    return SequentialSampler(dataset)


def build_tokenizer(config, model_config=None):
    """HF tokenizer of ``model.path`` when it is a directory with tokenizer files; integer tokenizer for presets.
    ``config`` is either the whole trainer config or a model section (``path`` / ``tokenizer_path``)."""
    from ..utils.tokenizer import IntTokenizer, hf_tokenizer
    from ..workers.engine_workers import resolve_model_config

    model = config.actor_rollout_ref.model if "actor_rollout_ref" in config else config
    trust = (config.get("data") or {}).get("trust_remote_code", False) if "actor_rollout_ref" in config else model.get(
        "trust_remote_code", False)
    path = os.path.expanduser(str(model.path))
    if os.path.isdir(path) and any(os.path.exists(os.path.join(path, f)) for f in ("tokenizer.json", "tokenizer_config.json")):
        return hf_tokenizer(model.get("tokenizer_path") or path, trust_remote_code=trust)
    mc = model_config if model_config is not None else resolve_model_config(model)[0]
    return IntTokenizer(mc.vocab_size, eos_token_id=mc.eos_token_id if mc.eos_token_id is not None else 2)


def run_ppo(config, spmd: Optional[bool] = None, trainer_cls=None, run_fit: bool = True):
    from ..workers.engine_workers import ActorRolloutRefWorker, CriticWorker, RewardModelWorker
    from .ppo.ray_trainer import RayPPOTrainer, ResourcePoolManager
    from .ppo.reward import load_reward_manager

    if spmd is None:
        spmd = int(os.environ.get("WORLD_SIZE", "1")) > 1 or os.environ.get("VERL_B200_SPMD") == "1"
    use_ref, use_critic = need_reference_policy(config), need_critic(config)
    validate_config(config, use_reference_policy=use_ref, use_critic=use_critic)
    tokenizer = build_tokenizer(config)
    mapping = {Role.ActorRollout: ActorRolloutRefWorker}
    pool_id = "global_pool"
    role_pool = {Role.ActorRollout: pool_id}
    if use_critic:
        mapping[Role.Critic] = CriticWorker
        role_pool[Role.Critic] = pool_id
    if config.reward_model.get("enable", False):
        mapping[Role.RewardModel] = RewardModelWorker
        role_pool[Role.RewardModel] = pool_id
    device = config.trainer.get("device", "cuda")
    n_gpus = [config.trainer.n_gpus_per_node] * config.trainer.nnodes
    if spmd:
        from ..single_controller.spmd import SPMDResourcePool, SPMDWorkerGroup

        rpm = ResourcePoolManager({pool_id: [1]}, role_pool, pool_cls=SPMDResourcePool, use_gpu=device == "cuda")
        wg_cls = SPMDWorkerGroup
    else:
        from ..single_controller.mp import MPWorkerGroup

        rpm = ResourcePoolManager({pool_id: n_gpus}, role_pool, use_gpu=device == "cuda")
        wg_cls = MPWorkerGroup
    reward_fn = load_reward_manager(config, tokenizer, num_examine=0)
    val_reward_fn = load_reward_manager(config, tokenizer, num_examine=1)
    train_ds = create_rl_dataset(config.data.train_files, config.data, tokenizer, is_train=True,
                                 max_samples=config.data.get("train_max_samples", -1))
    val_ds = None
    if config.data.get("val_files"):
        try:
            val_ds = create_rl_dataset(config.data.val_files, config.data, tokenizer, is_train=False,
                                       max_samples=config.data.get("val_max_samples", -1))
        except (FileNotFoundError, OSError):
            val_ds = None
    trainer = (trainer_cls or RayPPOTrainer)(config=config, tokenizer=tokenizer, role_worker_mapping=mapping, resource_pool_manager=rpm,
                            ray_worker_group_cls=wg_cls, reward_fn=reward_fn, val_reward_fn=val_reward_fn,
                            train_dataset=train_ds, val_dataset=val_ds, train_sampler=create_rl_sampler(config.data, train_ds),
                            device_name=device)
    trainer.init_workers()
    if not run_fit:
        return trainer  # the caller drives the steps (asynchronous pipelines) and calls trainer.shutdown()
    try:
        trainer.fit()
    finally:
        trainer.shutdown()
    return trainer


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    name = "ppo_trainer"
    for a in list(argv):
        if a.startswith("--config-name="):
            name = a.split("=", 1)[1]
            argv.remove(a)
    config = compose(name, argv)
    run_ppo(config)


if __name__ == "__main__":
    main()
