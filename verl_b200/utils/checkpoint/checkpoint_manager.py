"""Checkpoint bookkeeping shared by trainers: tracker file, latest-checkpoint discovery, rotation, ESI expiry
(verl/utils/checkpoint/checkpoint_manager.py:72-268)."""

from __future__ import annotations

import os
import re
import shutil
import tempfile
import time
from typing import Optional

TRACKER = "latest_checkpointed_iteration.txt"


def get_checkpoint_tracker_filename(root_path: str) -> str:
    return os.path.join(root_path, TRACKER)


def write_tracker(root_path: str, step: int) -> None:
    """Atomic update (write to a temp file, then rename)."""
    os.makedirs(root_path, exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=root_path, prefix=".tracker_")
    with os.fdopen(fd, "w") as f:
        f.write(str(step))
    os.replace(tmp, get_checkpoint_tracker_filename(root_path))


def find_latest_ckpt_path(path: Optional[str], directory_format: str = "global_step_{}") -> Optional[str]:
    if path is None:
        return None
    tracker = get_checkpoint_tracker_filename(path)
    if not os.path.exists(tracker):
        return None
    with open(tracker) as f:
        it = int(f.read().strip())
    ckpt = os.path.join(path, directory_format.format(it))
    if not os.path.exists(ckpt):
        print(f"Checkpoint does not exist: {ckpt}")
        return None
    print(f"Found checkpoint: {ckpt}")
    return ckpt


def list_checkpoints(root_path: str) -> list[tuple[int, str]]:
    out = []
    if not os.path.isdir(root_path):
        return out
    for name in os.listdir(root_path):
        m = re.fullmatch(r"global_step_(\d+)", name)
        if m:
            out.append((int(m.group(1)), os.path.join(root_path, name)))
    return sorted(out)


def rotate_checkpoints(root_path: str, max_to_keep: int) -> list[str]:
    """Delete the oldest ``global_step_*`` directories beyond ``max_to_keep``; returns what was removed."""
    removed = []
    ckpts = list_checkpoints(root_path)
    while max_to_keep > 0 and len(ckpts) > max_to_keep:
        _, old = ckpts.pop(0)
        shutil.rmtree(old, ignore_errors=True)
        removed.append(old)
    return removed


def should_save_ckpt_esi(max_steps_duration: float, save_ckpt_duration: float = 60, redundant_time: float = 0) -> bool:
    """True when a spot / pre-emptible instance is about to expire (expiry time from the environment) and
    there is just enough time left for one more step plus a checkpoint."""
    exp = os.getenv("MLP_CURRENT_CAPACITY_BLOCK_EXPIRATION_TIMESTAMP") or os.getenv("SAGEMAKER_CURRENT_CAPACITY_BLOCK_EXPIRATION_TIMESTAMP")
    if not exp:
        return False
    remaining = int(exp) - time.time()
    threshold = max_steps_duration + save_ckpt_duration + redundant_time
    return 0 < remaining <= threshold


class BaseCheckpointManager:
    """What a checkpoint manager of one model shares with every other (verl/utils/checkpoint/checkpoint_manager.py:32-178):
    which parts are saved / loaded (``checkpoint.save_contents`` / ``load_contents`` out of ``model``, ``optimizer``,
    ``extra``, ``hf_model``), the list of folders written by this run with removal of the oldest beyond
    ``max_ckpt_to_keep``, and the random-number-generator state. Subclasses write and read the files."""

    def __init__(self, model, optimizer=None, lr_scheduler=None, processing_class=None, checkpoint_config=None):
        get = (checkpoint_config.get if hasattr(checkpoint_config, "get") else
               (lambda k, d=None: getattr(checkpoint_config, k, d))) if checkpoint_config is not None else (lambda k, d=None: d)
        self.checkpoint_config = checkpoint_config
        self.checkpoint_load_contents = list(get("load_contents", None) or ["model", "optimizer", "extra"])
        self.checkpoint_save_contents = list(get("save_contents", None) or ["model", "optimizer", "extra"])
        self.model, self.optimizer, self.lr_scheduler, self.processing_class = model, optimizer, lr_scheduler, processing_class
        self.previous_global_step = None
        self.previous_saved_paths: list[str] = []
        import torch.distributed as dist

        on = dist.is_available() and dist.is_initialized()
        self.rank, self.world_size = (dist.get_rank(), dist.get_world_size()) if on else (0, 1)

    def __getattr__(self, name: str):
        # should_save_model / should_save_optimizer / should_save_extra / should_save_hf_model / should_load_...
        for verb in ("save", "load"):
            pre = f"should_{verb}_"
            if name.startswith(pre):
                return name[len(pre):] in self.__dict__.get(f"checkpoint_{verb}_contents", ())
        raise AttributeError(name)

    def load_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, del_local_after_load: bool = False):
        raise NotImplementedError

    def save_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, global_step: int = 0,
                        max_ckpt_to_keep: Optional[int] = None):
        raise NotImplementedError

    @staticmethod
    def checkpath(local_path: Optional[str], hdfs_path: Optional[str]):
        assert local_path is not None or hdfs_path is not None, "local_path and hdfs_path cannot be both None"
        return local_path is not None, local_path if local_path is not None else hdfs_path

    def remove_previous_save_local_path(self, path):
        import shutil

        for p in ([path] if isinstance(path, str) else list(path)):
            if os.path.isdir(os.path.abspath(p)):
                shutil.rmtree(os.path.abspath(p), ignore_errors=True)

    def ensure_checkpoint_capacity(self, max_ckpt_to_keep: Optional[int]) -> None:
        """Before a save: with ``max_ckpt_to_keep`` folders already written by this run, the oldest ones go."""
        if isinstance(max_ckpt_to_keep, int) and max_ckpt_to_keep > 0 and len(self.previous_saved_paths) >= max_ckpt_to_keep:
            n = len(self.previous_saved_paths) - max_ckpt_to_keep + 1
            self.remove_previous_save_local_path(self.previous_saved_paths[:n])
            self.previous_saved_paths = self.previous_saved_paths[n:]

    def register_checkpoint(self, new_path: str, max_ckpt_to_keep: Optional[int] = None) -> None:
        self.previous_saved_paths.append(new_path)

    @staticmethod
    def get_rng_state() -> dict:
        import random

        import numpy as np
        import torch

        st = {"cpu": torch.get_rng_state(), "numpy": np.random.get_state(), "random": random.getstate()}
        if torch.cuda.is_available():
            st["cuda"] = torch.cuda.get_rng_state()
        return st

    @staticmethod
    def load_rng_state(rng_state: dict) -> None:
        import random

        import numpy as np
        import torch

        torch.set_rng_state(rng_state["cpu"])
        np.random.set_state(rng_state["numpy"])
        random.setstate(rng_state["random"])
        if torch.cuda.is_available() and "cuda" in rng_state:
            torch.cuda.set_rng_state(rng_state["cuda"])


class NativeCheckpointManager(BaseCheckpointManager):
    """The manager of a :class:`~verl_b200.workers.engine.native.NativeEngine`: the engine writes and reads its shard
    files, this class applies the content lists, the retention limit and the remote copy."""

    def __init__(self, engine, processing_class=None, checkpoint_config=None):
        super().__init__(engine, None, None, processing_class, checkpoint_config)
        self.engine = engine

    def save_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, global_step: int = 0,
                        max_ckpt_to_keep: Optional[int] = None):
        import torch.distributed as dist

        from .native_checkpoint import save_engine_checkpoint

        if local_path is None:
            return
        self.previous_global_step = global_step
        if self.rank == 0:
            self.ensure_checkpoint_capacity(max_ckpt_to_keep)
        contents = tuple(c for c in self.checkpoint_save_contents if c != "hf_model")
        save_engine_checkpoint(self.engine, local_path, global_step=global_step, save_contents=contents)
        if dist.is_available() and dist.is_initialized() and self.world_size > 1:
            dist.barrier()
        if self.rank == 0:
            if hdfs_path:
                from .. import hdfs_io

                hdfs_io.makedirs(hdfs_path, exist_ok=True)
                hdfs_io.copy(src=local_path, dst=hdfs_path, dirs_exist_ok=True)
            self.register_checkpoint(local_path, max_ckpt_to_keep)

    def load_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, del_local_after_load: bool = False):
        from .native_checkpoint import load_engine_checkpoint

        if local_path is None:
            return
        load_engine_checkpoint(self.engine, local_path, load_contents=tuple(self.checkpoint_load_contents))
        if del_local_after_load and self.rank == 0:
            self.remove_previous_save_local_path(local_path)
