"""PPO / GRPO-family trainer: the controller loop.

Public surface of ``RayPPOTrainer`` (verl/trainer/ppo/ray_trainer.py:232-1721): the constructor signature,
``init_workers()``, ``fit()``, checkpoint / resume, validation, batch balancing, and the driver-side helpers
``apply_kl_penalty`` (:70), ``compute_response_mask`` (:112) and ``compute_advantage`` (:130).

Two launch modes share this loop:
  * single controller: this process holds the global batch and drives worker processes through a
    ``WorkerGroup`` (multiprocess backend by default);
  * SPMD (``torchrun``): every rank runs this loop on its own shard of each batch with an in-process
    worker group, and only scalars cross ranks. Batches then never pass through a driver.
"""

from __future__ import annotations

import json
import os
import time
import uuid
from collections import defaultdict
from contextlib import contextmanager
from copy import deepcopy
from pprint import pprint
from typing import Any, Optional

import numpy as np
import torch
import torch.distributed as dist

from ...protocol import DataProto, pad_dataproto_to_divisor, unpad_dataproto
from ...single_controller.base import ClassWithInitArgs
from ...utils.config import omega_conf_to_dataclass
from ...utils.seqlen_balancing import calculate_workload, get_seqlen_balanced_partitions, log_seqlen_unbalance
from ...utils.torch_functional import masked_mean
from . import core_algos
from .core_algos import AdvantageEstimator, agg_loss
from .metric_utils import (compute_data_metrics, compute_throughout_metrics, compute_timing_metrics,
                           compute_variance_proxy_metrics, process_validation_metrics, reduce_metrics)
from .reward import compute_reward, compute_reward_async
from .utils import Role, need_critic, need_reference_policy, need_reward_model

__all__ = ["RayPPOTrainer", "apply_kl_penalty", "compute_response_mask", "compute_advantage", "Role",
           "ResourcePoolManager"]


@contextmanager
def marked_timer(name: str, timing_raw: dict, color: Optional[str] = None):
    """Accumulate wall time of a stage into ``timing_raw[name]`` (verl/utils/profiler/performance.py:172)."""
    from ...utils.profiler.profile import nvtx_range

    t0 = time.perf_counter()
    with nvtx_range(name, color):
        yield
    timing_raw[name] = timing_raw.get(name, 0.0) + time.perf_counter() - t0


def apply_kl_penalty(data: DataProto, kl_ctrl, kl_penalty: str = "kl"):
    """token_level_rewards = token_level_scores - beta * KL(pi_old || pi_ref); updates the controller."""
    mask = data.batch["response_mask"]
    scores = data.batch["token_level_scores"]
    bs = data.batch.batch_size[0]
    kld = core_algos.kl_penalty(data.batch["old_log_probs"], data.batch["ref_log_prob"], kl_penalty=kl_penalty)
    kld = kld * mask
    beta = kl_ctrl.value
    data.batch["token_level_rewards"] = scores - beta * kld
    current_kl = torch.mean(masked_mean(kld, mask=mask, axis=-1), dim=0).item()
    kl_ctrl.update(current_kl=current_kl, n_steps=bs)
    return data, {"actor/reward_kl_penalty": current_kl, "actor/reward_kl_penalty_coeff": beta}


def compute_response_mask(data: DataProto) -> torch.Tensor:
    R = data.batch["responses"].size(1)
    return data.batch["attention_mask"][:, -R:]


def compute_advantage(data: DataProto, adv_estimator, gamma: float = 1.0, lam: float = 1.0, num_repeat: int = 1,
                      norm_adv_by_std_in_grpo: bool = True, config=None) -> DataProto:
    """Fill ``advantages`` and ``returns`` with the estimator named by ``adv_estimator``."""
    if "response_mask" not in data.batch.keys():
        data.batch["response_mask"] = compute_response_mask(data)
    name = adv_estimator.value if isinstance(adv_estimator, AdvantageEstimator) else adv_estimator
    b = data.batch
    if name == "gae":
        adv, ret = core_algos.compute_gae_advantage_return(b["token_level_rewards"], b["values"], b["response_mask"],
                                                           gamma, lam)
        if config is not None and config.get("use_pf_ppo", False):
            b["advantages"], b["returns"] = adv, ret
            pf = config.get("pf_ppo", {}) or {}
            return core_algos.compute_pf_ppo_reweight_data(data, pf.get("reweight_method", "pow"), pf.get("weight_pow", 2.0))
    elif name == "grpo":
        adv, ret = core_algos.compute_grpo_outcome_advantage(b["token_level_rewards"], b["response_mask"],
                                                             data.non_tensor_batch["uid"],
                                                             norm_adv_by_std_in_grpo=norm_adv_by_std_in_grpo)
    else:
        fn = core_algos.get_adv_estimator_fn(name)
        kw = {"token_level_rewards": b["token_level_rewards"], "response_mask": b["response_mask"], "config": config}
        if "uid" in data.non_tensor_batch:
            kw["index"] = data.non_tensor_batch["uid"]
        if "reward_baselines" in b.keys():
            kw["reward_baselines"] = b["reward_baselines"]
        if name in ("optimal_token_baseline", "tir_optimal_token_baseline"):
            assert "sum_pi_squared" in b.keys(), "set actor.calculate_sum_pi_squared=True for the optimal token baseline"
            kw.update(old_log_probs=b["old_log_probs"], sum_pi_squared=b["sum_pi_squared"],
                      rollout_is_weights=b.get("rollout_is_weights", None))
            kw.pop("config")
        adv, ret = fn(**kw)
    b["advantages"], b["returns"] = adv, ret
    return data


class ResourcePoolManager:
    """role -> resource pool. ``backend`` picks the worker-group implementation's pool class."""

    def __init__(self, resource_pool_spec: dict, mapping: dict, pool_cls=None, use_gpu: bool = True):
        self.resource_pool_spec, self.mapping, self.use_gpu = resource_pool_spec, mapping, use_gpu
        self.pool_cls = pool_cls
        self.resource_pool_dict: dict = {}

    def create_resource_pool(self):
        from ...single_controller.mp import MPResourcePool

        cls = self.pool_cls or MPResourcePool
        off = 0
        for name, nodes in self.resource_pool_spec.items():
            kw = {"gpu_offset": off} if cls is MPResourcePool else {}
            self.resource_pool_dict[name] = cls(process_on_nodes=nodes, use_gpu=self.use_gpu, max_colocate_count=3,
                                                name_prefix=name, **kw)
            off += sum(nodes)

    def get_resource_pool(self, role):
        return self.resource_pool_dict[self.mapping[role]]

    def get_n_gpus(self) -> int:
        return sum(n for nodes in self.resource_pool_spec.values() for n in nodes)


class _StatefulLoader:
    """DataLoader wrapper that can be checkpointed: remembers the epoch and how many batches were consumed
    (the role of torchdata's StatefulDataLoader in the reference, ray_trainer.py:314-394)."""

    def __init__(self, loader):
        self.loader = loader
        self.epoch, self.consumed = 0, 0
        self._skip = 0

    def __len__(self):
        return len(self.loader)

    def __iter__(self):
        skip, self._skip = self._skip, 0
        self.consumed = 0
        for i, batch in enumerate(self.loader):
            if i < skip:
                self.consumed += 1
                continue
            self.consumed += 1
            yield batch
        self.epoch += 1
        self.consumed = 0

    def state_dict(self):
        return {"epoch": self.epoch, "consumed": self.consumed}

    def load_state_dict(self, st):
        self.epoch, self._skip = int(st.get("epoch", 0)), int(st.get("consumed", 0))


def _wait_all(res):
    """Result of a non-blocking worker-group call: a future, or one future per worker. Waits for EVERY worker (the
    rollout servers take requests over HTTP, outside the workers' command queues, so a weight push still running on
    one worker must not overlap the next generation) and returns the first worker's value."""
    if hasattr(res, "result"):
        res = res.result()
    if isinstance(res, (list, tuple)):
        res = [r.result() if hasattr(r, "result") else r for r in res]
        res = res[0] if res else None
    return res


class RayPPOTrainer:
    def __init__(self, config, tokenizer, role_worker_mapping: dict, resource_pool_manager=None,
                 ray_worker_group_cls=None, processor=None, reward_fn=None, val_reward_fn=None, train_dataset=None,
                 val_dataset=None, collate_fn=None, train_sampler=None, device_name: Optional[str] = None):
        self.config = config
        self.tokenizer, self.processor = tokenizer, processor
        self.reward_fn, self.val_reward_fn = reward_fn, val_reward_fn
        self.role_worker_mapping = role_worker_mapping
        self.resource_pool_manager = resource_pool_manager
        if ray_worker_group_cls is None:
            from ...single_controller.mp import MPWorkerGroup as ray_worker_group_cls
        self.ray_worker_group_cls = ray_worker_group_cls
        self.spmd = bool(getattr(ray_worker_group_cls, "is_spmd", False))
        self.device_name = device_name or config.trainer.get("device", "cuda")
        self.hybrid_engine = config.actor_rollout_ref.hybrid_engine
        assert self.hybrid_engine, "Currently, only support hybrid engine"
        self.use_reference_policy = need_reference_policy(config)
        self.use_rm = need_reward_model(config)
        self.use_critic = need_critic(config)
        self.ref_in_actor = False
        self.validation_generations_logger = None
        if config.algorithm.get("use_kl_in_reward", False):
            self.kl_ctrl_in_reward = core_algos.get_kl_controller(config.algorithm.kl_ctrl)
        self.rank = dist.get_rank() if self.spmd and dist.is_initialized() else 0
        self.spmd_world = dist.get_world_size() if self.spmd and dist.is_initialized() else 1
        self.global_steps = 0
        self._create_dataloader(train_dataset, val_dataset, collate_fn, train_sampler)

    # ------------------------------------------------------------------ data
    def _create_dataloader(self, train_dataset, val_dataset, collate_fn, train_sampler):
        from torch.utils.data import DataLoader, RandomSampler, SequentialSampler

        from ...utils.dataset import RLHFDataset
        from ...utils.dataset import collate_fn as default_collate

        d = self.config.data
        if train_dataset is None:
            train_dataset = RLHFDataset(d.train_files, self.tokenizer, d, self.processor, d.get("train_max_samples", -1))
        if val_dataset is None and d.get("val_files"):
            try:
                val_dataset = RLHFDataset(d.val_files, self.tokenizer, d, self.processor, d.get("val_max_samples", -1))
            except (FileNotFoundError, OSError):
                val_dataset = None
        self.train_dataset, self.val_dataset = train_dataset, val_dataset
        collate_fn = collate_fn or default_collate
        if train_sampler is None:
            if d.get("shuffle", True):
                g = torch.Generator()
                g.manual_seed(int(d.get("seed") or 1))
                train_sampler = RandomSampler(train_dataset, generator=g)
            else:
                train_sampler = SequentialSampler(train_dataset)
        self.train_sampler = train_sampler
        self.train_dataloader = _StatefulLoader(DataLoader(
            train_dataset, batch_size=int(d.get("gen_batch_size", d.train_batch_size)), num_workers=0, drop_last=True,
            collate_fn=collate_fn, sampler=train_sampler))
        self.val_dataloader = None
        if val_dataset is not None and len(val_dataset) > 0:
            vbs = d.get("val_batch_size") or len(val_dataset)
            self.val_dataloader = DataLoader(val_dataset, batch_size=vbs, num_workers=0, shuffle=d.get("validation_shuffle", False),
                                             drop_last=False, collate_fn=collate_fn)
        assert len(self.train_dataloader) >= 1, "Train dataloader is empty!"
        total = len(self.train_dataloader) * self.config.trainer.total_epochs
        if self.config.trainer.get("total_training_steps") is not None:
            total = self.config.trainer.total_training_steps
        self.total_training_steps = total
        for node in (self.config.actor_rollout_ref.actor, self.config.critic):
            if node.get("optim") is not None:
                node.optim["total_training_steps"] = total

    # --------------------------------------------------------------- workers
    def init_workers(self):
        """Create worker groups (roles that share a pool are fused into one process per slot) and build models."""
        cfg = self.config
        if self.resource_pool_manager is not None:
            self.resource_pool_manager.create_resource_pool()
        pools: dict = defaultdict(dict)

        def pool_of(role):
            if self.resource_pool_manager is None:
                return None
            return self.resource_pool_manager.get_resource_pool(role)

        actor_role = Role.ActorRolloutRef if Role.ActorRolloutRef in self.role_worker_mapping else Role.ActorRollout
        role_name = "actor_rollout_ref" if actor_role == Role.ActorRolloutRef or (
            self.use_reference_policy and Role.RefPolicy not in self.role_worker_mapping) else "actor_rollout"
        if role_name == "actor_rollout_ref" and self.use_reference_policy:
            self.ref_in_actor = True
        pools[pool_of(actor_role)]["actor_rollout"] = ClassWithInitArgs(
            self.role_worker_mapping[actor_role], config=cfg.actor_rollout_ref,
            role=role_name if (self.use_reference_policy or actor_role == Role.ActorRolloutRef) else "actor_rollout",
            device_name=self.device_name)
        if self.use_critic:
            pools[pool_of(Role.Critic)]["critic"] = ClassWithInitArgs(self.role_worker_mapping[Role.Critic],
                                                                     config=cfg.critic, device_name=self.device_name)
        if self.use_reference_policy and not self.ref_in_actor:
            pools[pool_of(Role.RefPolicy)]["ref"] = ClassWithInitArgs(
                self.role_worker_mapping[Role.RefPolicy], config=cfg.actor_rollout_ref, role="ref", device_name=self.device_name)
        if self.use_rm and Role.RewardModel in self.role_worker_mapping:
            pools[pool_of(Role.RewardModel)]["rm"] = ClassWithInitArgs(
                self.role_worker_mapping[Role.RewardModel], config=cfg.reward_model, device_name=self.device_name)

        all_wg: dict = {}
        self._wg_roots = []
        for pool, class_dict in pools.items():
            if self.spmd:
                from ...single_controller.spmd import create_colocated_worker_cls_spmd as fuse
            else:
                from ...single_controller.mp import create_colocated_worker_cls as fuse
            fused = fuse(class_dict)
            kw = {} if self.spmd else {"device_name": self.device_name}
            root = self.ray_worker_group_cls(resource_pool=pool, ray_cls_with_init=fused, **kw)
            self._wg_roots.append(root)
            all_wg.update(root.spawn(prefix_set=class_dict.keys()))
        if self.use_critic:
            self.critic_wg = all_wg["critic"]
            self.critic_wg.init_model()
        if self.use_reference_policy and not self.ref_in_actor:
            self.ref_policy_wg = all_wg["ref"]
            self.ref_policy_wg.init_model()
        self.rm_wg = None
        if "rm" in all_wg:
            self.rm_wg = all_wg["rm"]
            self.rm_wg.init_model()
        self.actor_rollout_wg = all_wg["actor_rollout"]
        self.actor_rollout_wg.init_model()
        if self.ref_in_actor:
            self.ref_policy_wg = self.actor_rollout_wg
        self.async_rollout_mode = False
        rc = self.config.actor_rollout_ref.rollout
        agent = rc.get("agent") or {}
        if (bool((rc.get("multi_turn") or {}).get("enable", False)) or bool(agent.get("use_agent_loop", False))
                or agent.get("default_agent_loop", "single_turn_agent") not in (None, "single_turn_agent")):
            self._init_async_rollout_manager()
        self.n_gpus = (self.spmd_world if self.spmd else
                       (self.resource_pool_manager.get_n_gpus() if self.resource_pool_manager else 1))

    def _init_async_rollout_manager(self):
        """Rollouts through agent loops (multi-turn, tools, interactions) instead of one batched ``generate`` call:
        role of ``AgentLoopManager`` in the reference's ``rollout.mode=async``. Taken when ``rollout.multi_turn.enable``
        is set, a non-default agent loop is configured, or ``rollout.agent.use_agent_loop`` is true; plain single-turn
        RL keeps the batched path (same continuous batching, no per-request hand-off)."""
        from ...experimental.agent_loop import AgentLoopManager

        if self.spmd:
            if int(self.config.actor_rollout_ref.rollout.get("tensor_model_parallel_size", 1) or 1) > 1:
                raise ValueError("rollouts through the agent loops with rollout.tensor_model_parallel_size > 1 need the "
                                 "dispatching worker group (one driver that owns the replicas' endpoints); under an SPMD "
                                 "launch every rank drives its own requests. Use the batched rollout or TP = 1.")
            worker = self.actor_rollout_wg.worker.worker_dict["actor_rollout"]
            handles = [worker.get_async_server()]
        else:
            from ...workers.rollout.async_server import HttpServerHandle

            # one endpoint per replica: the followers of a tensor-parallel replica answer with an empty address
            handles = [HttpServerHandle(a) for a in self.actor_rollout_wg.start_rollout_server() if a]
        self.async_rollout_manager = AgentLoopManager(self.config, server_handles=handles, tokenizer=self.tokenizer,
                                                      processor=self.processor)
        self._rollout_server_handles = handles
        self.async_rollout_mode = True

    def _generate(self, gen_batch: DataProto) -> DataProto:
        """One rollout of ``gen_batch`` (already repeated n times): agent loops or the batched engine call."""
        if self.async_rollout_mode:
            import asyncio

            free = bool(self.config.actor_rollout_ref.rollout.get("free_cache_engine", True))

            async def run():
                await asyncio.gather(*[h.wake_up() for h in self._rollout_server_handles])
                out = await self.async_rollout_manager.generate_sequences_async(gen_batch)
                if free and not gen_batch.meta_info.get("keep_cache", False):
                    await asyncio.gather(*[h.sleep() for h in self._rollout_server_handles])
                for h in self._rollout_server_handles:
                    if hasattr(h, "close"):
                        await h.close()
                return out

            out = asyncio.run(run())
            timing = out.meta_info.pop("timing", {})
            out.meta_info["metrics"] = {k: float(v) for k, v in timing.items()}
            return out
        div = 1 if self.spmd else self.actor_rollout_wg.world_size
        padded, pad = pad_dataproto_to_divisor(gen_batch, div)
        return unpad_dataproto(self.actor_rollout_wg.generate_sequences(padded), pad_size=pad)

    def shutdown(self):
        for root in getattr(self, "_wg_roots", []):
            root.shutdown()

    # ------------------------------------------------------------ small helpers
    def _local(self, batch: DataProto) -> DataProto:
        """SPMD mode: this rank's contiguous share of a global batch (groups of n samples stay together)."""
        if not self.spmd or self.spmd_world == 1:
            return batch
        return batch.chunk(self.spmd_world)[self.rank]

    def _all_reduce_metrics(self, metrics: dict) -> dict:
        """SPMD mode: average scalar metrics over ranks (max / min keys use max / min)."""
        if not self.spmd or self.spmd_world == 1:
            return metrics
        keys = sorted(k for k, v in metrics.items() if isinstance(v, (int, float)))
        gathered = [None] * self.spmd_world
        dist.all_gather_object(gathered, {k: float(metrics[k]) for k in keys})
        out = dict(metrics)
        for k in keys:
            vals = [g[k] for g in gathered if k in g]
            if "max" in k:
                out[k] = max(vals)
            elif "min" in k:
                out[k] = min(vals)
            elif k in ("perf/total_num_tokens",):
                out[k] = sum(vals)
            else:
                out[k] = float(np.mean(vals))
        return out

    def _get_gen_batch(self, batch: DataProto) -> DataProto:
        """Move the prompt tensors out of ``batch`` (the rollout returns the full-length versions)."""
        keys = [k for k in ("input_ids", "attention_mask", "position_ids") if k in batch.batch.keys()]
        nt = [k for k in ("raw_prompt_ids", "raw_prompt", "tools_kwargs", "interaction_kwargs", "agent_name")
              if k in batch.non_tensor_batch]
        gen = batch.pop(batch_keys=keys, non_tensor_batch_keys=nt)
        if "multi_modal_inputs" in batch.non_tensor_batch:  # images: the rollout needs them, the actor too (kept)
            gen.non_tensor_batch["multi_modal_inputs"] = batch.non_tensor_batch["multi_modal_inputs"]
        if batch.batch is not None and len(list(batch.batch.keys())) == 0:
            batch.batch = None
        return gen

    # --------------------------------------------------------------- validation
    def _validate(self) -> dict:
        if self.val_dataloader is None or self.val_reward_fn is None:
            return {}
        rewards, sources, uids = [], [], []
        extra_infos: dict = defaultdict(list)
        inputs, outputs = [], []
        for test_data in self.val_dataloader:
            test_batch = self._local(DataProto.from_single_dict(test_data))
            n = int(self.config.actor_rollout_ref.rollout.val_kwargs.n)
            if "uid" not in test_batch.non_tensor_batch:
                test_batch.non_tensor_batch["uid"] = np.array([str(uuid.uuid4()) for _ in range(len(test_batch))], dtype=object)
            test_batch = test_batch.repeat(repeat_times=n, interleave=True)
            gen = self._get_gen_batch(test_batch)
            vk = self.config.actor_rollout_ref.rollout.val_kwargs
            gen.meta_info.update({"eos_token_id": getattr(self.tokenizer, "eos_token_id", None),
                                  "pad_token_id": getattr(self.tokenizer, "pad_token_id", 0) or 0, "recompute_log_prob": False,
                                  "do_sample": vk.do_sample, "validate": True, "global_steps": self.global_steps})
            out = self._generate(gen)
            for k in list(out.non_tensor_batch.keys()):
                if k in test_batch.non_tensor_batch:
                    out.non_tensor_batch.pop(k)
            test_batch = test_batch.union(out)
            test_batch.meta_info["validate"] = True
            res = self.val_reward_fn(test_batch, return_dict=True)
            score = res["reward_tensor"].sum(-1).cpu().tolist()
            rewards.extend(score)
            extra_infos["reward"].extend(score)
            for k, v in res.get("reward_extra_info", {}).items():
                extra_infos[k].extend(list(v))
            sources.extend(list(test_batch.non_tensor_batch.get("data_source", ["unknown"] * len(score))))
            uids.extend(list(test_batch.non_tensor_batch["uid"]))
            if self.config.trainer.get("log_val_generations", 0) > 0:
                P = test_batch.batch["prompts"].shape[-1]
                for i in range(min(len(test_batch), self.config.trainer.log_val_generations - len(inputs))):
                    inputs.append(self.tokenizer.decode(test_batch.batch["prompts"][i], skip_special_tokens=True))
                    outputs.append(self.tokenizer.decode(test_batch.batch["responses"][i], skip_special_tokens=True))
        if inputs:
            from ...utils.tracking import ValidationGenerationsLogger

            ValidationGenerationsLogger(self.config.trainer.project_name, self.config.trainer.experiment_name).log(
                self.config.trainer.logger, list(zip(inputs, outputs, rewards[: len(inputs)])), self.global_steps)
        per = process_validation_metrics(sources, uids, dict(extra_infos))
        metrics = {}
        for ds, vars_ in per.items():
            core_var = "acc" if "acc" in vars_ else "reward"
            for var, mets in vars_.items():
                n_max = max(int(name.split("@")[-1].split("/")[0]) for name in mets)
                for name, v in mets.items():
                    core = (var == core_var and any(name.startswith(p) for p in ("mean", "maj", "best"))
                            and f"@{n_max}" in name)
                    metrics[f"{'val-core' if core else 'val-aux'}/{ds}/{var}/{name}"] = v
        return self._all_reduce_metrics(metrics)

    # --------------------------------------------------------------- checkpoint
    def _ckpt_dir(self) -> str:
        return os.path.expanduser(self.config.trainer.default_local_dir)

    def _save_checkpoint(self):
        """``{default_local_dir}/global_step_{N}/{actor,critic}/...`` + ``data.pt`` + tracker file."""
        from ...utils.checkpoint.checkpoint_manager import rotate_checkpoints, write_tracker

        step_dir = os.path.join(self._ckpt_dir(), f"global_step_{self.global_steps}")
        print(f"local_global_step_folder: {step_dir}")
        tr = self.config.trainer
        self.actor_rollout_wg.save_checkpoint(os.path.join(step_dir, "actor"), None, self.global_steps,
                                              tr.get("max_actor_ckpt_to_keep"))
        if self.use_critic:
            self.critic_wg.save_checkpoint(os.path.join(step_dir, "critic"), None, self.global_steps,
                                           tr.get("max_critic_ckpt_to_keep"))
        if self.rank == 0:
            os.makedirs(step_dir, exist_ok=True)
            torch.save(self.train_dataloader.state_dict(), os.path.join(step_dir, "data.pt"))
            write_tracker(self._ckpt_dir(), self.global_steps)
            keep = tr.get("max_actor_ckpt_to_keep")
            if keep:
                rotate_checkpoints(self._ckpt_dir(), int(keep))
        if self.spmd and self.spmd_world > 1:
            dist.barrier()

    def _load_checkpoint(self) -> int:
        from ...utils.checkpoint.checkpoint_manager import find_latest_ckpt_path

        tr = self.config.trainer
        mode = tr.get("resume_mode", "auto")
        if mode == "disable":
            return 0
        folder = None
        if mode == "resume_path":
            folder = tr.get("resume_from_path")
            assert folder and "global_step_" in folder, "resume ckpt must specify the global_steps"
            if not os.path.isabs(folder):
                folder = os.path.join(os.getcwd(), folder)
        else:
            folder = find_latest_ckpt_path(self._ckpt_dir())
        if folder is None:
            print("Training from scratch")
            return 0
        print(f"Load from checkpoint folder: {folder}")
        self.global_steps = int(folder.split("global_step_")[-1].rstrip("/"))
        dl = tr.get("del_local_ckpt_after_load", False)
        self.actor_rollout_wg.load_checkpoint(os.path.join(folder, "actor"), None, dl)
        if self.use_critic:
            self.critic_wg.load_checkpoint(os.path.join(folder, "critic"), None, dl)
        data_pt = os.path.join(folder, "data.pt")
        if os.path.exists(data_pt):
            self.train_dataloader.load_state_dict(torch.load(data_pt, weights_only=False))
        else:
            print(f"Warning: No dataloader state found at {data_pt}, will start from scratch")
        return self.global_steps

    # ---------------------------------------------------------------- balancing
    def _balance_batch(self, batch: DataProto, metrics: dict, logging_prefix: str = "global_seqlen"):
        """Reorder the batch so every data-parallel rank receives a similar number of tokens."""
        world = 1 if self.spmd else self.actor_rollout_wg.world_size
        if world <= 1:
            return
        lens = batch.batch["attention_mask"].view(len(batch), -1).sum(-1)
        work = calculate_workload(lens).tolist()
        parts = get_seqlen_balanced_partitions(work, k_partitions=world, equal_size=True)
        for p in parts:  # small-large-small order inside a partition helps micro-batch packing
            p.sort(key=lambda i: (work[i], i))
            p[:] = p[::2] + p[1::2][::-1]
        idx = torch.tensor([j for p in parts for j in p])
        batch.reorder(idx)
        metrics.update(log_seqlen_unbalance(lens.tolist(), parts, logging_prefix))

    # ----------------------------------------------------------------- the step
    def _filter_groups(self, batch: DataProto, metric_name: str) -> DataProto:
        """Dynamic sampling (DAPO): drop prompt groups whose metric is identical over all samples."""
        if metric_name == "seq_final_reward":
            vals = batch.batch["token_level_rewards"].sum(-1).numpy()
        elif metric_name == "seq_reward":
            vals = batch.batch["token_level_scores"].sum(-1).numpy()
        else:
            vals = np.asarray(batch.non_tensor_batch[metric_name], dtype=np.float64)
        by_uid: dict = defaultdict(list)
        for uid, v in zip(batch.non_tensor_batch["uid"], vals):
            by_uid[uid].append(v)
        keep_uid = {u for u, vs in by_uid.items() if np.std(vs) > 0 or len(vs) == 1}
        keep = [i for i, u in enumerate(batch.non_tensor_batch["uid"]) if u in keep_uid]
        return batch[keep]

    def _rollout_and_reward(self, batch_dict: dict, timing_raw: dict, metrics: dict) -> DataProto:
        cfg = self.config
        n = int(cfg.actor_rollout_ref.rollout.n)
        batch = self._local(DataProto.from_single_dict(batch_dict))
        batch.non_tensor_batch["uid"] = np.array([str(uuid.uuid4()) for _ in range(len(batch))], dtype=object)
        gen_batch = self._get_gen_batch(batch)
        gen_batch.meta_info.update({"global_steps": self.global_steps, "pad_token_id": getattr(self.tokenizer, "pad_token_id", 0) or 0,
                                    "eos_token_id": getattr(self.tokenizer, "eos_token_id", None)})
        gen_batch = gen_batch.repeat(repeat_times=n, interleave=True)
        with marked_timer("gen", timing_raw, "red"):
            gen_out = self._generate(gen_batch)
            for k, v in (gen_out.meta_info.pop("metrics", {}) or {}).items():
                metrics[k] = float(np.mean(v)) if isinstance(v, list) else v
        if cfg.algorithm.adv_estimator == "remax":
            with marked_timer("gen_max", timing_raw, "purple"):
                base = deepcopy(gen_batch)
                base.meta_info["do_sample"] = False
                base_out = self._generate(base)
                tmp = batch.repeat(repeat_times=n, interleave=True).union(base_out)
                rb, _ = compute_reward(tmp, self.reward_fn)
                batch_baseline = rb.sum(dim=-1)
        batch = batch.repeat(repeat_times=n, interleave=True)
        batch = self._attach_rollout_and_reward(batch, gen_out, timing_raw)
        if cfg.algorithm.adv_estimator == "remax":
            batch.batch["reward_baselines"] = batch_baseline
        return batch

    def _attach_rollout_and_reward(self, batch: DataProto, gen_out: DataProto, timing_raw: dict) -> DataProto:
        """``batch`` (prompt-side fields, already repeated n times) + rollout output -> batch with
        ``token_level_scores``. Also used by producers that generate elsewhere (streaming rollouter)."""
        for k in list(gen_out.non_tensor_batch.keys()):
            if k in batch.non_tensor_batch:
                gen_out.non_tensor_batch.pop(k)
        batch = batch.union(gen_out)
        if "response_mask" not in batch.batch.keys():
            batch.batch["response_mask"] = compute_response_mask(batch)
        with marked_timer("reward", timing_raw, "yellow"):
            if self.use_rm and "rm_scores" not in batch.batch.keys() and self.rm_wg is not None:
                batch = batch.union(self.rm_wg.compute_rm_score(batch))
            fg = self.config.algorithm.get("filter_groups") or {}
            rm_cfg = self.config.get("reward_model") or {}
            if bool(rm_cfg.get("launch_reward_fn_async", False)) and not fg.get("enable", False):
                # the rule-based reward runs on a host thread while the GPUs compute the log-probs; joined before the
                # advantages (reward_model.launch_reward_fn_async of the reference, verl/trainer/ppo/ray_trainer.py).
                # Dynamic sampling needs the scores at once and keeps the synchronous path.
                # Rows must not be permuted after this point, so the sequence-length
                # balancing of the batch happens now instead of at the start of the training part.
                if self.config.trainer.get("balance_batch", True):
                    self._balance_batch(batch, {})
                    batch.meta_info["batch_balanced"] = True
                if not hasattr(self, "_reward_futures"):
                    self._reward_futures = {}
                # kept on the trainer (a future cannot travel to worker processes), keyed by the batch's first sample
                self._reward_futures[str(batch.non_tensor_batch["uid"][0])] = compute_reward_async(batch, reward_fn=self.reward_fn)
                return batch
            self._attach_reward(batch, *compute_reward(batch, self.reward_fn))
        return batch

    @staticmethod
    def _attach_reward(batch: DataProto, reward_tensor, extra) -> None:
        batch.batch["token_level_scores"] = reward_tensor
        if extra:
            batch.non_tensor_batch.update({k: np.array(v, dtype=object) for k, v in extra.items() if len(v) == len(batch)})

    def _join_reward(self, batch: DataProto, timing_raw: dict) -> None:
        fut = getattr(self, "_reward_futures", {}).pop(str(batch.non_tensor_batch["uid"][0]), None) \
            if "uid" in batch.non_tensor_batch else None
        if fut is not None:
            with marked_timer("reward_wait", timing_raw, "yellow"):
                self._attach_reward(batch, *fut.result())

    def train_step(self, batch_dict: dict) -> dict:
        """One RL step on one (global, or per-rank in SPMD mode) batch of prompts. Returns the step's metrics.

        With dynamic sampling (``algorithm.filter_groups``) a batch whose kept groups do not fill the train batch is
        held back and the call returns ``{"train/accumulating": 1.0, ...}`` without training and without advancing
        ``global_steps``; the following calls add their kept groups until the batch is full
        (verl/recipe dapo_ray_trainer: ``continue`` in the batch loop)."""
        metrics: dict = {}
        timing_raw: dict = {}
        self.global_steps += 1
        with marked_timer("step", timing_raw):
            batch = self._rollout_and_reward(batch_dict, timing_raw, metrics)
            batch = self._dynamic_sampling(batch, metrics)
            if batch is None:
                self.global_steps -= 1
                metrics["train/accumulating"] = 1.0
                return metrics
            self._train_on_batch(batch, timing_raw, metrics)
        return self._finish_step(timing_raw, metrics)

    def _dynamic_sampling(self, batch: DataProto, metrics: dict) -> Optional[DataProto]:
        """DAPO dynamic sampling: keep the prompt groups whose metric varies, accumulate them over generation batches
        until ``train_batch_size`` prompts are there. Returns the batch to train on, or None while accumulating.
        Raises once ``max_num_gen_batches`` generation batches were not enough."""
        cfg = self.config
        fg = cfg.algorithm.get("filter_groups") or {}
        if not fg.get("enable", False):
            return batch
        n = int(cfg.actor_rollout_ref.rollout.n)
        want = (len(batch) // n) * n
        batch.batch["token_level_rewards"] = batch.batch["token_level_scores"]
        kept = self._filter_groups(batch, fg.get("metric") or "seq_reward")
        pending = getattr(self, "_fg_pending", None)
        if pending is not None and len(pending):
            kept = DataProto.concat([pending, kept])
        self._fg_tries = getattr(self, "_fg_tries", 0) + 1
        metrics["train/num_gen_batches"] = self._fg_tries
        if len(kept) < want:
            max_tries = int(fg.get("max_num_gen_batches", 0) or 0)
            if max_tries > 0 and self._fg_tries >= max_tries:
                self._fg_pending, self._fg_tries = None, 0
                raise ValueError(f"dynamic sampling: {max_tries} generation batches gave {len(kept) // n} of "
                                 f"{want // n} prompt groups with a varying {fg.get('metric') or 'seq_reward'}; "
                                 "the data is too easy or too hard, or raise algorithm.filter_groups.max_num_gen_batches")
            self._fg_pending = kept
            return None
        self._fg_pending, self._fg_tries = None, 0
        return kept[:want]

    def _train_on_batch(self, batch: DataProto, timing_raw: dict, metrics: dict) -> None:
        """Everything after rollout + reward (+ dynamic sampling): log-probs, advantages, critic / actor update, weight
        sync. Split out so that asynchronous trainers can feed batches produced elsewhere."""
        cfg = self.config
        if True:
            if cfg.trainer.get("balance_batch", True) and not batch.meta_info.pop("batch_balanced", False):
                self._balance_batch(batch, metrics)
            batch.meta_info["global_token_num"] = torch.sum(batch.batch["attention_mask"], dim=-1).tolist()
            # under an SPMD launch every rank drives the trainer on its own shard of the batch: the token list is
            # already per rank and must not be divided by the world size again (MFU)
            batch.meta_info["token_num_is_local"] = self.spmd
            batch.meta_info["temperature"] = cfg.actor_rollout_ref.rollout.temperature

            rc = cfg.algorithm.get("rollout_correction") or {}
            bypass = bool(rc.get("bypass_mode", False))
            if bypass:
                from .rollout_corr_helper import apply_bypass_mode

                apply_bypass_mode(batch, rc, cfg.actor_rollout_ref.actor.policy_loss)
            else:
                with marked_timer("old_log_prob", timing_raw, "blue"):
                    old = self.actor_rollout_wg.compute_log_prob(batch)
                    ent = old.batch["entropys"]
                    mask = batch.batch["response_mask"]
                    metrics["actor/entropy"] = agg_loss(ent, mask, cfg.actor_rollout_ref.actor.loss_agg_mode).item()
                    old.batch.pop("entropys")
                    batch = batch.union(old)
                    if "rollout_log_probs" in batch.batch.keys():
                        from ...utils.debug import calculate_debug_metrics

                        metrics.update(calculate_debug_metrics(batch))
            if self.use_reference_policy:
                with marked_timer("ref", timing_raw, "olive"):
                    batch = batch.union(self.ref_policy_wg.compute_ref_log_prob(batch))
            if self.use_critic:
                with marked_timer("values", timing_raw, "cyan"):
                    batch = batch.union(self.critic_wg.compute_values(batch))
            self._join_reward(batch, timing_raw)
            with marked_timer("adv", timing_raw, "brown"):
                if cfg.algorithm.get("use_kl_in_reward", False):
                    batch, kl_m = apply_kl_penalty(batch, self.kl_ctrl_in_reward, cfg.algorithm.kl_penalty)
                    metrics.update(kl_m)
                else:
                    batch.batch["token_level_rewards"] = batch.batch["token_level_scores"]
                if (rc.get("rollout_is") or rc.get("rollout_rs")) and not bypass and "rollout_log_probs" in batch.batch.keys():
                    from .rollout_corr_helper import compute_rollout_correction_and_add_to_batch

                    batch, rc_m = compute_rollout_correction_and_add_to_batch(batch, rc)
                    metrics.update(rc_m)
                batch = compute_advantage(batch, cfg.algorithm.adv_estimator, cfg.algorithm.gamma, cfg.algorithm.lam,
                                          int(cfg.actor_rollout_ref.rollout.n), cfg.algorithm.get("norm_adv_by_std_in_grpo", True),
                                          cfg.algorithm)
            if self.use_critic:
                with marked_timer("update_critic", timing_raw, "pink"):
                    out = self.critic_wg.update_critic(batch)
                metrics.update(reduce_metrics(out.meta_info["metrics"]))
            if cfg.trainer.get("critic_warmup", 0) <= self.global_steps:
                with marked_timer("update_actor", timing_raw, "red"):
                    out = self.actor_rollout_wg.update_actor(batch)
                metrics.update(reduce_metrics(out.meta_info["metrics"]))
                with marked_timer("update_weights", timing_raw, "red"):
                    res = _wait_all(self.actor_rollout_wg.update_weights(self.global_steps))
                    if isinstance(res, dict) and "resync_s" in res:
                        metrics["timing_s/resync"] = res["resync_s"]
            dump_dir = cfg.trainer.get("rollout_data_dir")
            if dump_dir:
                self._dump_generations(batch, dump_dir)
        self._last_batch = batch

    def _finish_step(self, timing_raw: dict, metrics: dict) -> dict:
        batch = self._last_batch
        metrics.update(compute_data_metrics(batch, use_critic=self.use_critic))
        metrics.update(compute_timing_metrics(batch, timing_raw))
        n_gpus = 1 if self.spmd else self.n_gpus
        metrics.update(compute_throughout_metrics(batch, timing_raw, n_gpus))
        metrics.update(compute_variance_proxy_metrics(batch, metrics.get("actor/grad_norm")))
        metrics["training/global_step"] = self.global_steps
        self._last_batch = batch
        if hasattr(getattr(self, "train_sampler", None), "update"):  # curriculum samplers learn from the finished batch
            self.train_sampler.update(batch=batch)
        if hasattr(getattr(self, "train_dataset", None), "on_batch_end"):  # datasets that grow during training
            self.train_dataset.on_batch_end(batch=batch)
        return self._all_reduce_metrics(metrics)

    def _dump_generations(self, batch: DataProto, dump_dir: str):
        os.makedirs(dump_dir, exist_ok=True)
        path = os.path.join(dump_dir, f"{self.global_steps}.jsonl" if self.spmd_world == 1 else f"{self.global_steps}_rank{self.rank}.jsonl")
        scores = batch.batch["token_level_scores"].sum(-1).tolist()
        with open(path, "w") as f:
            for i in range(len(batch)):
                f.write(json.dumps({"input": self.tokenizer.decode(batch.batch["prompts"][i], skip_special_tokens=True),
                                    "output": self.tokenizer.decode(batch.batch["responses"][i], skip_special_tokens=True),
                                    "score": scores[i], "step": self.global_steps}) + "\n")

    # ---------------------------------------------------------------------- fit
    def fit(self):
        from ...utils.checkpoint.checkpoint_manager import should_save_ckpt_esi
        from ...utils.tracking import Tracking
        from ...utils.config import to_container

        cfg = self.config
        tr = cfg.trainer
        logger = None
        if self.rank == 0:
            logger = Tracking(tr.project_name, tr.experiment_name, list(tr.logger), config=to_container(cfg))
        self.global_steps = 0
        self._load_checkpoint()
        _wait_all(self.actor_rollout_wg.update_weights(self.global_steps))
        if self.val_reward_fn is not None and tr.get("val_before_train", True):
            val_metrics = self._validate()
            if val_metrics and logger is not None:
                pprint(f"Initial validation metrics: {val_metrics}")
                logger.log(data=val_metrics, step=self.global_steps)
            if tr.get("val_only", False):
                return
        last_val = None
        max_step_time = 0.0
        prof_steps = set((cfg.get("global_profiler") or {}).get("steps") or [])
        for epoch in range(self.train_dataloader.epoch, tr.total_epochs):
            for batch_dict in self.train_dataloader:
                do_prof = (self.global_steps + 1) in prof_steps
                if do_prof:
                    self.actor_rollout_wg.start_profile(role="e2e", profile_step=self.global_steps + 1)
                metrics = self.train_step(batch_dict)
                if do_prof:
                    self.actor_rollout_wg.stop_profile()
                if metrics.get("train/accumulating"):
                    continue  # dynamic sampling wants another generation batch before this step can train
                is_last = self.global_steps >= self.total_training_steps
                if self.val_reward_fn is not None and tr.test_freq > 0 and (is_last or self.global_steps % tr.test_freq == 0):
                    last_val = self._validate()
                    metrics.update(last_val)
                max_step_time = max(max_step_time, metrics.get("timing_s/step", 0.0))
                esi = should_save_ckpt_esi(max_step_time, redundant_time=tr.get("esi_redundant_time", 0))
                if tr.save_freq > 0 and (is_last or self.global_steps % tr.save_freq == 0 or esi):
                    if esi:
                        print("Force saving checkpoint: ESI instance expiration approaching.")
                    t0 = time.perf_counter()
                    self._save_checkpoint()
                    metrics["timing_s/save_checkpoint"] = time.perf_counter() - t0
                if logger is not None:
                    logger.log(data=metrics, step=self.global_steps)
                if is_last:
                    if last_val:
                        pprint(f"Final validation metrics: {last_val}")
                    return
