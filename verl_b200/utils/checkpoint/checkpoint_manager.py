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
