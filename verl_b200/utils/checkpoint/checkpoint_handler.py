"""Checkpoint orchestration for a single-model trainer (role of verl/utils/checkpoint/checkpoint_handler.py:32-225): owns the
``global_step_N`` folder naming, the tracker file, rotation, the per-data-parallel-rank loader state and the choice of
the folder to resume from. The engine writes and reads its own shards."""

from __future__ import annotations

import os
import re
from enum import Enum
from typing import Optional

import torch
import torch.distributed as dist

from .. import hdfs_io
from .checkpoint_manager import find_latest_ckpt_path, rotate_checkpoints, write_tracker

_STEP = re.compile(r"global_step_(\d+)")


def extract_step(path: str) -> Optional[int]:
    m = _STEP.search(path or "")
    return int(m.group(1)) if m else None


class OrchestrationMode(Enum):
    SPMD = 0  # one process per GPU; this object lives in every rank
    RAY = 1  # a single controller that drives a worker group


class CheckpointHandler:
    def __init__(self, engine, train_dataloader, *, default_local_dir: str, max_ckpt_to_keep: Optional[int] = None,
                 default_hdfs_dir: Optional[str] = None, resume_mode: str = "auto", resume_from_path: Optional[str] = None,
                 mode: OrchestrationMode = OrchestrationMode.SPMD):
        self.engine, self.train_dataloader, self.mode = engine, train_dataloader, mode
        self.default_local_dir = os.path.expanduser(default_local_dir)
        self.max_ckpt_to_keep, self.default_hdfs_dir = max_ckpt_to_keep, default_hdfs_dir
        self.resume_mode, self.resume_from_path = resume_mode, resume_from_path
        self.resume_global_step = 0
        if mode == OrchestrationMode.SPMD:
            self.rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
            self.is_mp_src_rank_with_outputs = bool(engine.is_mp_src_rank_with_outputs())
            self.dp_rank = int(engine.get_data_parallel_rank())
        else:  # the controller holds the (identical across ranks) loader state
            self.rank, self.is_mp_src_rank_with_outputs, self.dp_rank = 0, True, 0

    # ------------------------------------------------------------------ save
    def save_checkpoint(self, step: int) -> str:
        folder = os.path.join(self.default_local_dir, f"global_step_{step}")
        self.engine.save_checkpoint(local_path=folder, global_step=step, max_ckpt_to_keep=self.max_ckpt_to_keep)
        if self.is_mp_src_rank_with_outputs and hasattr(self.train_dataloader, "state_dict"):
            os.makedirs(folder, exist_ok=True)
            torch.save(self.train_dataloader.state_dict(), os.path.join(folder, f"data_{self.dp_rank}.pt"))
        self._barrier()
        if self.rank == 0:
            write_tracker(self.default_local_dir, step)  # written last, atomically: a crash before it leaves the old one
            if self.max_ckpt_to_keep:
                rotate_checkpoints(self.default_local_dir, int(self.max_ckpt_to_keep))
            if self.default_hdfs_dir:
                hdfs_io.makedirs(self.default_hdfs_dir, exist_ok=True)
                hdfs_io.copy(src=folder, dst=self.default_hdfs_dir, dirs_exist_ok=True)
        self._barrier()
        return folder

    # ------------------------------------------------------------------ load
    def load_checkpoint(self) -> int:
        """Loads model / optimizer / loader state from the folder the resume mode selects; returns its step (0: none)."""
        path = self._determine_resume_path()
        step = extract_step(path) if path else None
        if step is None:
            return 0
        self.resume_global_step = step
        self.engine.load_checkpoint(path)
        data = os.path.join(path, f"data_{self.dp_rank}.pt")
        if os.path.exists(data) and hasattr(self.train_dataloader, "load_state_dict"):
            self.train_dataloader.load_state_dict(torch.load(data, map_location="cpu", weights_only=False))
        return step

    def _determine_resume_path(self) -> Optional[str]:
        mode, path = self.resume_mode, self.resume_from_path
        if mode == "disable":
            return None
        if mode not in ("auto", "resume_path"):
            raise ValueError(f"Invalid resume_mode: {mode}. Must be 'auto', 'disable', or 'resume_path'")
        if mode == "resume_path" or path is not None:
            assert path and os.path.exists(path), "resume_from_path must be an existing path"
            assert "global_step_" in path, "resume_from_path must specify the global_steps"
            return path
        return find_latest_ckpt_path(self.default_local_dir) if os.path.isdir(self.default_local_dir) else None

    def _barrier(self):
        if self.mode == OrchestrationMode.SPMD and dist.is_available() and dist.is_initialized():
            dist.barrier()
