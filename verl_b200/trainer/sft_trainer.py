"""Supervised fine-tuning, SPMD (one process per GPU, torchrun or a single process).

    python -m verl_b200.trainer.sft_trainer data.train_files=... model.path=preset:qwen2.5-0.5b
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m verl_b200.trainer.sft_trainer ...

Role of verl/trainer/sft_trainer.py:60-421 (``SFTTrainer``: dataset + stateful loader + engine + checkpoint
handler; ``fit`` = forward_backward over dynamic micro-batches, optimizer step, metric all-reduce, validation,
save). The loss is the token-mean negative log-likelihood over ``loss_mask``; log-probs come from the fused
lm_head kernel, so the ``[tokens, vocab]`` logits never exist.
"""

from __future__ import annotations

import math
import os
import sys
import time
from typing import Optional

import torch
import torch.distributed as dist

from ..models.transformer import PackedBatch
from ..utils import tracking
from ..utils.checkpoint.checkpoint_manager import find_latest_ckpt_path, rotate_checkpoints, write_tracker
from ..utils.config import compose
from ..utils.dataset.sft_dataset import MultiTurnSFTDataset, SFTDataset, sft_collate_fn
from ..utils.seqlen_balancing import ceildiv, get_seqlen_balanced_partitions
from ..workers.engine.native import NativeEngine
from ..workers.engine_workers import resolve_model_config
from ..workers.utils.losses import sft_loss


def _g(c, k, d=None):
    v = c.get(k, d) if hasattr(c, "get") else getattr(c, k, d)
    return d if v is None else v


class SFTTrainer:
    def __init__(self, config, tokenizer=None, train_dataset=None, val_dataset=None):
        self.config = config
        self.rank = int(os.environ.get("RANK", 0))
        self.world = int(os.environ.get("WORLD_SIZE", 1))
        dev = _g(config.trainer, "device", "cuda")
        if dev == "cuda" and not torch.cuda.is_available():
            dev = "cpu"
        if dev == "cuda":
            self.device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
            torch.cuda.set_device(self.device)
        else:
            self.device = torch.device("cpu")
        if self.world > 1 and not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl" if self.device.type == "cuda" else "gloo")
        self.group = dist.group.WORLD if self.world > 1 else None
        torch.manual_seed(int(_g(config.trainer, "seed", 1)))

        model_cfg, state = resolve_model_config(config.model)
        self.model_config = model_cfg
        if tokenizer is None:
            from .main_ppo import build_tokenizer

            tokenizer = build_tokenizer(config.model, model_cfg)
        self.tokenizer = tokenizer
        self.train_dataset = train_dataset or self._build_dataset(config.data.train_files, _g(config.data, "train_max_samples", -1))
        vf = _g(config.data, "val_files")
        self.val_dataset = val_dataset or (self._build_dataset(vf, _g(config.data, "val_max_samples", -1)) if vf else None)

        bs = int(config.data.train_batch_size)
        assert bs % self.world == 0, "data.train_batch_size must be divisible by the number of ranks"
        self.local_bs = bs // self.world
        self.steps_per_epoch = len(self.train_dataset) // bs
        total = _g(config.trainer, "total_training_steps")
        self.total_steps = int(total) if total else self.steps_per_epoch * int(config.trainer.total_epochs)
        optim = config.optim
        if hasattr(optim, "total_training_steps"):
            try:
                optim.total_training_steps = self.total_steps
            except Exception:
                pass
        comm = None
        if self.device.type == "cuda" and self.world > 1 and not os.environ.get("VERL_B200_DISABLE_PEER_COMM"):
            try:
                from ..parallel.peer_comm import PeerComm

                comm = PeerComm(dist.group.WORLD)
            except Exception:
                comm = None
        self.engine = NativeEngine(model_cfg, config.engine, optim, device=str(self.device), group=self.group,
                                   seed=int(_g(config.engine, "seed", 42)), state_dict=state, comm=comm,
                                   gradient_checkpointing=bool(_g(config.model, "enable_gradient_checkpointing", True)),
                                   lora=({"rank": int(_g(config.model, "lora_rank", 0) or 0),
                                          "alpha": _g(config.model, "lora_alpha", 16),
                                          "target_modules": _g(config.model, "target_modules", "all-linear"),
                                          "exclude_modules": _g(config.model, "exclude_modules", None)}
                                         if int(_g(config.model, "lora_rank", 0) or 0) > 0 else None)).initialize()
        self.global_step = 0
        self.logger = None
        self._resume()

    # ------------------------------------------------------------------ data
    def _build_dataset(self, files, max_samples):
        d = self.config.data
        cls = MultiTurnSFTDataset if _g(d, "multiturn", True) else SFTDataset
        custom = _g(d, "custom_cls")
        if custom and _g(custom, "path"):
            from ..utils.py_functional import load_extern_object

            cls = load_extern_object(custom.path, custom.name)
        return cls(files, self.tokenizer, d, max_samples=max_samples)

    def _epoch_indices(self, epoch: int) -> list[int]:
        n = len(self.train_dataset)
        if _g(self.config.data, "shuffle", True):
            g = torch.Generator().manual_seed(int(_g(self.config.trainer, "seed", 1)) + epoch)
            return torch.randperm(n, generator=g).tolist()
        return list(range(n))

    def _batches(self, start_step: int):
        """Yield (epoch, [dataset indices of this rank]) from ``start_step`` on; every rank derives the same global
        order, so resuming needs only the step counter."""
        bs = int(self.config.data.train_batch_size)
        step = 0
        for epoch in range(int(self.config.trainer.total_epochs) + 1):
            order = self._epoch_indices(epoch)
            for b in range(self.steps_per_epoch):
                if step >= start_step:
                    glob = order[b * bs : (b + 1) * bs]
                    yield epoch, glob[self.rank * self.local_bs : (self.rank + 1) * self.local_bs]
                step += 1
                if step >= self.total_steps:
                    return

    # ------------------------------------------------------------------ step
    def _micro_batches(self, batch: dict) -> list[torch.Tensor]:
        d = self.config.data
        n = batch["input_ids"].shape[0]
        if _g(d, "use_dynamic_bsz", True):
            lens = batch["attention_mask"].sum(-1).tolist()
            num = min(n, max(1, ceildiv(int(sum(lens)), int(d.max_token_len_per_gpu))))
            if self.world > 1:  # every rank runs the same number of micro-batches (the collectives are per unit call)
                t = torch.tensor([num], device=self.device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
                num = min(n, int(t.item()))
            parts = get_seqlen_balanced_partitions(lens, num, equal_size=False)
            return [torch.tensor(sorted(p), dtype=torch.long) for p in parts]
        m = int(d.micro_batch_size_per_gpu)
        return [torch.arange(i, min(i + m, n)) for i in range(0, n, m)]

    def _forward(self, batch: dict, idx: torch.Tensor):
        dev = self.device
        ids = batch["input_ids"][idx].to(dev, non_blocking=True)
        attn = batch["attention_mask"][idx].to(dev, non_blocking=True)
        loss_mask = batch["loss_mask"][idx].to(dev, non_blocking=True) * attn
        packed, flat = PackedBatch.from_padded(ids, attn, batch["position_ids"][idx].to(dev) if "position_ids" in batch else None)
        B, S = ids.shape
        inv = torch.full((B * S,), -1, dtype=torch.long, device=dev)
        inv[flat] = torch.arange(flat.numel(), device=dev)
        # position (b, s) with loss predicts token (b, s + 1)
        bs_idx = torch.nonzero(loss_mask[:, :-1].bool() & attn[:, 1:].bool(), as_tuple=False)
        rows = inv[bs_idx[:, 0] * S + bs_idx[:, 1]]
        labels = ids[bs_idx[:, 0], bs_idx[:, 1] + 1]
        lp, _ = self.engine.forward_logprob(packed, rows, labels, 1.0)
        return lp

    def train_step(self, batch: dict) -> dict:
        eng = self.engine
        t0 = time.perf_counter()
        local_tokens = float((batch["loss_mask"][:, :-1] * batch["attention_mask"][:, 1:]).sum())
        tok = torch.tensor([local_tokens, float(batch["attention_mask"].sum())], dtype=torch.float64, device=self.device)
        if self.world > 1:
            dist.all_reduce(tok, group=self.group)
        global_tokens = float(tok[0])
        loss_sum = torch.zeros((), dtype=torch.float32, device=self.device)
        with eng.train_mode():
            eng.optimizer_zero_grad()
            for idx in self._micro_batches(batch):
                lp = self._forward(batch, idx)
                # gradients are summed over ranks: dividing by the global token count gives the global token mean
                loss = -lp.sum() / max(global_tokens, 1.0)
                loss.backward()
                loss_sum += loss.detach()
            grad_norm = eng.optimizer_step()
            lr = eng.lr_scheduler_step()
        if self.world > 1:
            dist.all_reduce(loss_sum, group=self.group)
        dt = time.perf_counter() - t0
        return {"train/loss": float(loss_sum), "train/grad_norm": float(grad_norm), "train/lr": float(lr),
                "train/global_tokens": float(tok[1]), "train/time_per_step": dt,
                "perf/tokens_per_s": float(tok[1]) / max(dt, 1e-9)}

    @torch.no_grad()
    def validate(self) -> dict:
        if self.val_dataset is None:
            return {}
        n = len(self.val_dataset)
        mine = list(range(self.rank, n, self.world))
        m = int(self.config.data.micro_batch_size_per_gpu)
        acc = torch.zeros(2, dtype=torch.float64, device=self.device)
        with self.engine.eval_mode():
            for i in range(0, len(mine), m):
                batch = sft_collate_fn([self.val_dataset[j] for j in mine[i : i + m]])
                lp = self._forward(batch, torch.arange(batch["input_ids"].shape[0]))
                acc[0] += -lp.double().sum()
                acc[1] += lp.numel()
        if self.world > 1:
            dist.all_reduce(acc, group=self.group)
        return {"val/loss": float(acc[0] / acc[1].clamp(min=1))}

    # ------------------------------------------------------------ checkpoints
    def _ckpt_root(self) -> str:
        return os.path.expanduser(str(self.config.trainer.default_local_dir))

    def _resume(self):
        mode = _g(self.config.trainer, "resume_mode", "auto")
        if mode == "disable":
            return
        path = _g(self.config.trainer, "resume_from_path") if mode == "resume_path" else find_latest_ckpt_path(self._ckpt_root())
        if not path or not os.path.isdir(path):
            return
        self.engine.load_checkpoint(path, load_contents=tuple(_g(self.config.checkpoint, "load_contents", ("model", "optimizer", "extra"))))
        self.global_step = int(os.path.basename(path.rstrip("/")).split("_")[-1])
        self.engine.lr_step = self.global_step
        if self.rank == 0:
            print(f"[sft] resumed from {path} at step {self.global_step}")

    def save_checkpoint(self):
        root = self._ckpt_root()
        path = os.path.join(root, f"global_step_{self.global_step}")
        self.engine.save_checkpoint(path, global_step=self.global_step,
                                    save_contents=tuple(_g(self.config.checkpoint, "save_contents", ("model", "optimizer", "extra"))))
        if self.world > 1:
            dist.barrier(group=self.group)
        if self.rank == 0:
            write_tracker(root, self.global_step)
            keep = _g(self.config.trainer, "max_ckpt_to_keep")
            if keep:
                rotate_checkpoints(root, int(keep))

    # -------------------------------------------------------------------- fit
    def fit(self) -> dict:
        cfg = self.config
        if self.rank == 0 and self.logger is None:
            self.logger = tracking.Tracking(project_name=cfg.trainer.project_name, experiment_name=cfg.trainer.experiment_name,
                                            default_backend=list(_g(cfg.trainer, "logger", ["console"])), config=None)
        save_freq, test_freq = int(_g(cfg.trainer, "save_freq", -1)), int(_g(cfg.trainer, "test_freq", -1))
        last = {}
        for _, indices in self._batches(self.global_step):
            batch = sft_collate_fn([self.train_dataset[i] for i in indices])
            metrics = self.train_step(batch)
            self.global_step += 1
            is_last = self.global_step >= self.total_steps
            if test_freq > 0 and (is_last or self.global_step % test_freq == 0):
                metrics.update(self.validate())
            if save_freq > 0 and (is_last or self.global_step % save_freq == 0):
                self.save_checkpoint()
            if self.logger is not None:
                self.logger.log(metrics, step=self.global_step)
            last = metrics
            if is_last or not math.isfinite(metrics["train/loss"]):
                break
        return last


def run_sft(config) -> dict:
    trainer = SFTTrainer(config)
    out = trainer.fit()
    if dist.is_initialized():
        dist.barrier()
    return out


def main(argv: Optional[list[str]] = None):
    overrides = list(sys.argv[1:] if argv is None else argv)
    config = compose("sft_trainer", overrides)
    run_sft(config)


if __name__ == "__main__":
    main()
