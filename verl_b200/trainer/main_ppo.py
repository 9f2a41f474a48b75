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
        # with a vision-language processor and data.synthetic_image_size > 0 every prompt carries one random image
        parts = data_paths.split(":")
        num, lo, hi, id_lo, id_hi, seed = (int(x) for x in parts[1:7])
        source = parts[7] if len(parts) > 7 else "synthetic/even_fraction"
        gt = int(parts[8]) if len(parts) > 8 else None
        return SyntheticPromptDataset(num, lo, hi, id_lo, id_hi, data_config.max_prompt_length, seed, source,
                                      getattr(tokenizer, "pad_token_id", 0) or 0, gt, processor=processor,
                                      image_size=int(data_config.get("synthetic_image_size", 0) or 0),
                                      video_frames=int(data_config.get("synthetic_video_frames", 0) or 0))
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
        tok = hf_tokenizer(model.get("tokenizer_path") or path, trust_remote_code=trust)
        if model.get("custom_chat_template", None) is not None:  # model.custom_chat_template replaces the checkpoint's
            tok.chat_template = model.get("custom_chat_template")
        return tok
    mc = model_config if model_config is not None else resolve_model_config(model)[0]
    return IntTokenizer(mc.vocab_size, eos_token_id=mc.eos_token_id if mc.eos_token_id is not None else 2)


def build_processor(config, model_config=None):
    """Multimodal processor of the policy model (None for text-only models)."""
    from ..utils.dataset.vision_utils import VLProcessor
    from ..workers.engine_workers import resolve_model_config

    model = config.actor_rollout_ref.model if "actor_rollout_ref" in config else config
    mc = model_config if model_config is not None else resolve_model_config(model)[0]
    return VLProcessor.from_model_config(mc)


class TaskRunner:
    """Builds the role -> worker mapping, the resource pools, datasets and reward managers, then runs the trainer
    (the extension point of verl/trainer/main_ppo.py:108-368: subclass it and override a step to plug in other
    workers, pools or trainers; ``run_ppo(config, task_runner_class=...)`` uses the subclass)."""

    trainer_cls = None  # default: RayPPOTrainer

    def __init__(self):
        self.role_worker_mapping: dict = {}
        self.mapping: dict = {}  # role -> resource pool id
        self.pool_id = "global_pool"

    # ---------------------------------------------------------------- workers
    def add_actor_rollout_worker(self, config):
        from ..workers.engine_workers import ActorRolloutRefWorker

        self.role_worker_mapping[Role.ActorRollout] = ActorRolloutRefWorker
        self.mapping[Role.ActorRollout] = self.pool_id
        return ActorRolloutRefWorker

    def add_critic_worker(self, config):
        from ..workers.engine_workers import CriticWorker

        if need_critic(config):
            self.role_worker_mapping[Role.Critic] = CriticWorker
            self.mapping[Role.Critic] = self.pool_id

    def add_reward_model_worker(self, config):
        from ..workers.engine_workers import RewardModelWorker

        if config.reward_model.get("enable", False):
            self.role_worker_mapping[Role.RewardModel] = RewardModelWorker
            self.mapping[Role.RewardModel] = self.pool_id

    def add_ref_policy_worker(self, config, ref_policy_cls=None):
        """The reference policy lives inside the actor worker (``actor_rollout_ref``) unless a class is given."""
        if ref_policy_cls is not None and need_reference_policy(config):
            self.role_worker_mapping[Role.RefPolicy] = ref_policy_cls
            self.mapping[Role.RefPolicy] = self.pool_id

    def init_resource_pool_mgr(self, config, spmd: bool):
        from .ppo.ray_trainer import ResourcePoolManager

        device = config.trainer.get("device", "cuda")
        if spmd:
            from ..single_controller.spmd import SPMDResourcePool, SPMDWorkerGroup

            return (ResourcePoolManager({self.pool_id: [1]}, self.mapping, pool_cls=SPMDResourcePool, use_gpu=device == "cuda"),
                    SPMDWorkerGroup)
        from ..single_controller.mp import MPWorkerGroup

        n_gpus = [config.trainer.n_gpus_per_node] * config.trainer.nnodes
        return ResourcePoolManager({self.pool_id: n_gpus}, self.mapping, use_gpu=device == "cuda"), MPWorkerGroup

    # -------------------------------------------------------------------- run
    def run(self, config, spmd: Optional[bool] = None, trainer_cls=None, run_fit: bool = True):
        from .ppo.ray_trainer import RayPPOTrainer
        from .ppo.reward import load_reward_manager

        if spmd is None:
            spmd = int(os.environ.get("WORLD_SIZE", "1")) > 1 or os.environ.get("VERL_B200_SPMD") == "1"
        use_ref, use_critic = need_reference_policy(config), need_critic(config)
        validate_config(config, use_reference_policy=use_ref, use_critic=use_critic)
        tokenizer = build_tokenizer(config)
        processor = build_processor(config)
        self.add_actor_rollout_worker(config)
        self.add_critic_worker(config)
        self.add_reward_model_worker(config)
        self.add_ref_policy_worker(config)
        rpm, wg_cls = self.init_resource_pool_mgr(config, spmd)
        reward_fn = load_reward_manager(config, tokenizer, num_examine=0)
        val_reward_fn = load_reward_manager(config, tokenizer, num_examine=1)
        train_ds = create_rl_dataset(config.data.train_files, config.data, tokenizer, processor, is_train=True,
                                     max_samples=config.data.get("train_max_samples", -1))
        val_ds = None
        if config.data.get("val_files"):
            try:
                val_ds = create_rl_dataset(config.data.val_files, config.data, tokenizer, processor, is_train=False,
                                           max_samples=config.data.get("val_max_samples", -1))
            except (FileNotFoundError, OSError):
                val_ds = None
        cls = trainer_cls or self.trainer_cls or RayPPOTrainer
        trainer = cls(config=config, tokenizer=tokenizer, role_worker_mapping=self.role_worker_mapping,
                      resource_pool_manager=rpm, ray_worker_group_cls=wg_cls, reward_fn=reward_fn, val_reward_fn=val_reward_fn,
                      train_dataset=train_ds, val_dataset=val_ds, train_sampler=create_rl_sampler(config.data, train_ds),
                      device_name=config.trainer.get("device", "cuda"))
        trainer.init_workers()
        if not run_fit:
            return trainer  # the caller drives the steps (asynchronous pipelines) and calls trainer.shutdown()
        try:
            trainer.fit()
        finally:
            trainer.shutdown()
        return trainer


def run_ppo(config, spmd: Optional[bool] = None, trainer_cls=None, run_fit: bool = True, task_runner_class=None):
    return (task_runner_class or TaskRunner)().run(config, spmd=spmd, trainer_cls=trainer_cls, run_fit=run_fit)


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    name, rest, it = "ppo_trainer", [], iter(argv)
    for a in it:
        # Hydra's launcher flags: --config-name[=]NAME[.yaml] (ppo_megatron_trainer maps onto the one engine, see
        # utils.config.translate_megatron_overrides); --config-path is not needed (the tree ships with the package)
        if a.startswith("--config-name"):
            name = (a.split("=", 1)[1] if "=" in a else next(it)).strip("'\"")
            name = name[: -len(".yaml")] if name.endswith(".yaml") else name
        elif a.startswith("--config-path"):
            if "=" not in a:
                next(it, None)
        else:
            rest.append(a)
    config = compose(name, rest)
    run_ppo(config)


if __name__ == "__main__":
    main()
