"""Supervised fine-tuning driven by a single controller (role of verl/trainer/sft_trainer_ray.py:48-362).

The controller owns the dataset, the batch order and the checkpoint bookkeeping; a worker group of
:class:`~verl_b200.workers.training_worker.TrainingWorker` (one process per GPU) owns the sharded model. Every step
the controller sends ONE TensorDict in the no-padding layout (``input_ids`` / ``loss_mask`` / ``position_ids`` as jagged
nested tensors); the group's dispatch hands each data-parallel rank its share and ``train_batch`` does the
micro-batching, the gradient reduction and the optimizer step. ``python -m verl_b200.trainer.sft_trainer_ray`` takes the
overrides of the SPMD trainer (``verl_b200.trainer.sft_trainer``, one process per GPU under torchrun, no controller).
"""

from __future__ import annotations

import os
import sys
import time
from functools import partial
from typing import Optional

import torch

from ..utils import tensordict_utils as tu
from ..utils import tracking
from ..utils.checkpoint.checkpoint_handler import CheckpointHandler, OrchestrationMode
from ..utils.config import compose
from ..utils.dataset.sft_dataset import MultiTurnSFTDataset, SFTDataset
from ..workers.utils.losses import sft_loss_on_batch


def _g(c, k, d=None):
    v = c.get(k, d) if hasattr(c, "get") else getattr(c, k, d)
    return d if v is None else v


class StatefulBatchSampler:
    """Global batches of dataset indices, epoch after epoch (a seeded permutation per epoch). The state is the number of
    batches already handed out, so a resumed run continues with the batch that follows the checkpointed one (the
    ``StatefulDataLoader`` state of the reference's trainer)."""

    def __init__(self, n: int, batch_size: int, total_epochs: int, shuffle: bool = True, seed: int = 1):
        self.n, self.bs, self.epochs, self.shuffle, self.seed = n, batch_size, total_epochs, shuffle, seed
        self.steps_per_epoch = n // batch_size
        self.step = 0

    def state_dict(self) -> dict:
        return {"step": self.step}

    def load_state_dict(self, sd: dict) -> None:
        self.step = int(sd["step"])

    def _order(self, epoch: int) -> list[int]:
        if not self.shuffle:
            return list(range(self.n))
        return torch.randperm(self.n, generator=torch.Generator().manual_seed(self.seed + epoch)).tolist()

    def __iter__(self):
        while self.step < self.steps_per_epoch * self.epochs:
            epoch, b = divmod(self.step, self.steps_per_epoch)
            order = self._order(epoch)
            self.step += 1
            yield order[b * self.bs : (b + 1) * self.bs]


def to_no_padding_batch(items: list[dict], meta: dict):
    """Dataset rows (padded or ragged, with ``attention_mask``) -> TensorDict of jagged nested tensors + the knobs."""
    nt = lambda xs: torch.nested.as_nested_tensor(xs, layout=torch.jagged)  # noqa: E731
    keep = [it["attention_mask"].bool() if "attention_mask" in it else torch.ones_like(it["input_ids"], dtype=torch.bool)
            for it in items]
    tensors = {"input_ids": nt([it["input_ids"][k] for it, k in zip(items, keep)]),
               "loss_mask": nt([it["loss_mask"][k] for it, k in zip(items, keep)])}
    if "position_ids" in items[0]:
        tensors["position_ids"] = nt([it["position_ids"][..., k] for it, k in zip(items, keep)])
    return tu.get_tensordict(tensors, dict(meta))


class SFTTrainer:
    def __init__(self, config, tokenizer=None, train_dataset=None, val_dataset=None):
        self.config = config
        t = config.trainer
        self.device_name = _g(t, "device", "cuda")
        if self.device_name == "cuda" and not torch.cuda.is_available():
            self.device_name = "cpu"
        self.world = int(_g(t, "n_gpus_per_node", 1)) * int(_g(t, "nnodes", 1))
        if tokenizer is None:
            from .main_ppo import build_tokenizer

            tokenizer = build_tokenizer(config.model)
        self.tokenizer = tokenizer
        d = config.data
        self.train_dataset = train_dataset or self._build_dataset(d.train_files, _g(d, "train_max_samples", -1))
        vf = _g(d, "val_files")
        self.val_dataset = val_dataset or (self._build_dataset(vf, _g(d, "val_max_samples", -1)) if vf else None)
        self.global_batch_size = int(d.train_batch_size)
        assert self.global_batch_size % self.world == 0, "data.train_batch_size must be divisible by the number of workers"
        self.train_dataloader = StatefulBatchSampler(len(self.train_dataset), self.global_batch_size, int(t.total_epochs),
                                                     bool(_g(d, "shuffle", True)), int(_g(t, "seed", 1)))
        total = _g(t, "total_training_steps")
        self.total_training_steps = int(total) if total else self.train_dataloader.steps_per_epoch * int(t.total_epochs)
        try:
            config.optim.total_training_steps = self.total_training_steps
        except Exception:
            pass
        self.save_freq, self.test_freq = int(_g(t, "save_freq", -1)), int(_g(t, "test_freq", -1))
        self.profile_interval = tuple(_g(t, "profile_interval", (-1, -1)))
        self._build_engine()
        self.ckpt_handler = CheckpointHandler(
            engine=self.training_client, train_dataloader=self.train_dataloader, default_local_dir=t.default_local_dir,
            max_ckpt_to_keep=_g(t, "max_ckpt_to_keep"), default_hdfs_dir=_g(t, "default_hdfs_dir"),
            resume_mode=_g(t, "resume_mode", "auto"), resume_from_path=_g(t, "resume_from_path"), mode=OrchestrationMode.RAY)
        self.resume_global_step = self.ckpt_handler.load_checkpoint()

    # ------------------------------------------------------------------ parts
    def _build_dataset(self, files, max_samples):
        d = self.config.data
        cls = MultiTurnSFTDataset if _g(d, "multiturn", True) else SFTDataset
        custom = _g(d, "custom_cls")
        if custom and _g(custom, "path"):
            from ..utils.py_functional import load_extern_object

            cls = load_extern_object(custom.path, custom.name)
        return cls(files, self.tokenizer, d, max_samples=max_samples)

    def _build_engine(self):
        from ..single_controller.ray import RayClassWithInitArgs, RayResourcePool, RayWorkerGroup
        from ..workers.training_worker import TrainingWorker

        c, t = self.config, self.config.trainer
        worker_cfg = {"model_type": "language_model", "model_config": c.model, "engine_config": c.engine,
                      "optimizer_config": c.optim, "checkpoint_config": _g(c, "checkpoint")}
        pool = RayResourcePool(process_on_nodes=[int(_g(t, "n_gpus_per_node", 1))] * int(_g(t, "nnodes", 1)),
                               use_gpu=self.device_name == "cuda")
        cls = RayClassWithInitArgs(TrainingWorker, config=worker_cfg, device_name=self.device_name)
        self.resource_pool = pool
        self.training_client = RayWorkerGroup(resource_pool=pool, ray_cls_with_init=cls, device_name=self.device_name)
        self.training_client.set_loss_fn(partial(sft_loss_on_batch, None))
        self.training_client.reset()

    def _meta(self) -> dict:
        d = self.config.data
        return {"use_dynamic_bsz": bool(_g(d, "use_dynamic_bsz", True)), "max_token_len_per_gpu": int(d.max_token_len_per_gpu),
                "micro_batch_size_per_gpu": int(d.micro_batch_size_per_gpu), "temperature": 1.0,
                "global_batch_size": self.global_batch_size}

    @staticmethod
    def _get(out):
        return out.get() if hasattr(out, "get") and not hasattr(out, "keys") else out

    # -------------------------------------------------------------------- steps
    def train_step(self, indices: list[int]) -> dict:
        data = to_no_padding_batch([self.train_dataset[i] for i in indices], self._meta())
        seqlens = data["input_ids"].offsets().diff().tolist()
        tu.assign_non_tensor_data(data, "global_token_num", seqlens)
        tu.assign_non_tensor_data(data, "update_lr_scheduler", True)
        t0 = time.perf_counter()
        m = dict(tu.get(self._get(self.training_client.train_batch(data)), "metrics"))
        dt = time.perf_counter() - t0
        tokens = float(sum(seqlens))
        out = {"train/loss": float(m.pop("loss")), "train/grad_norm": float(m.pop("grad_norm")), "train/lr": float(m.pop("lr", 0.0)),
               "train/mfu": float(m.pop("mfu", 0.0)), "train/global_tokens": tokens, "train/time_per_step": dt,
               "perf/tokens_per_s": tokens / max(dt, 1e-9)}
        return out

    def validate(self) -> dict:
        if self.val_dataset is None:
            return {}
        n, losses = len(self.val_dataset), []
        bs = max(self.world, int(self.config.data.micro_batch_size_per_gpu) * self.world)
        for i in range(0, n - n % self.world, bs):
            idx = list(range(i, min(i + bs, n - n % self.world)))
            data = to_no_padding_batch([self.val_dataset[j] for j in idx], self._meta())
            tokens = float(sum(float(self.val_dataset[j]["loss_mask"].sum()) for j in idx))
            out = tu.get(self._get(self.training_client.infer_batch(data)), "metrics")
            losses.append((float(out["loss"]), tokens))
        total = sum(t for _, t in losses)
        return {"val/loss": sum(l * t for l, t in losses) / max(total, 1.0)} if losses else {}

    # ---------------------------------------------------------------------- fit
    def fit(self) -> dict:
        cfg = self.config
        logger = tracking.Tracking(project_name=cfg.trainer.project_name, experiment_name=cfg.trainer.experiment_name,
                                   default_backend=list(_g(cfg.trainer, "logger", ["console"])), config=None)
        step, last, total_tokens = self.resume_global_step, {}, 0.0
        for indices in self.train_dataloader:
            step += 1
            if step == self.profile_interval[0]:
                self.training_client.start_profile()
            metrics = self.train_step(indices)
            if step == self.profile_interval[1]:
                self.training_client.stop_profile()
            total_tokens += metrics["train/global_tokens"]
            metrics["train/total_tokens(B)"] = total_tokens / 1e9
            is_last = step >= self.total_training_steps
            if self.val_dataset is not None and (is_last or (self.test_freq > 0 and step % self.test_freq == 0)):
                metrics.update(self.validate())
            if is_last or (self.save_freq > 0 and step % self.save_freq == 0):
                self.ckpt_handler.save_checkpoint(step)
            logger.log(metrics, step=step)
            last = metrics
            if is_last:
                break
        self.global_step = step
        return last

    def shutdown(self):
        if hasattr(self.training_client, "shutdown"):
            self.training_client.shutdown()


def run_sft(config) -> dict:
    trainer = SFTTrainer(config)
    try:
        return trainer.fit()
    finally:
        trainer.shutdown()


def main(argv: Optional[list[str]] = None):
    overrides = list(sys.argv[1:] if argv is None else argv)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    run_sft(compose("sft_trainer", overrides))


if __name__ == "__main__":
    main()
