"""Dump intermediate tensors of a run for offline comparison (verl/utils/debug/trajectory_tracker.py:34-110).

Enabled by ``VERL_ENABLE_TRACKER=1`` with ``VERL_TRACKER_HDFS_DIR`` naming the target directory (a local or mounted
path; ``hdfs://`` URLs go through :mod:`verl_b200.utils.hdfs_io`). Writes happen on a background thread pool so that the
training step does not wait for storage."""

from __future__ import annotations

import io
import os
import tempfile
from concurrent.futures import ThreadPoolExecutor

import torch

from ..hdfs_io import copy as _copy
from ..hdfs_io import makedirs as _makedirs

_TRACKER = None


def save_to_hdfs(data: io.BytesIO, name: str, hdfs_dir: str, verbose: bool) -> None:
    filename = name + ".pth"
    with tempfile.TemporaryDirectory() as tmp:
        local = os.path.join(tmp, filename)
        with open(local, "wb") as f:
            f.write(data.getbuffer())
        _makedirs(hdfs_dir, exist_ok=True)
        _copy(local, os.path.join(hdfs_dir, filename))
        if verbose:
            print(f"Saved {local} to {hdfs_dir}")


class TrajectoryTracker:
    def __init__(self, hdfs_dir: str, verbose: bool = False) -> None:
        self.hdfs_dir, self.verbose = hdfs_dir, verbose
        self.pool = ThreadPoolExecutor(max_workers=2)
        self.handles = []

    def dump(self, data: io.BytesIO, name: str) -> None:
        self.handles.append(self.pool.submit(save_to_hdfs, data, name, self.hdfs_dir, self.verbose))

    def wait_for_hdfs(self) -> None:
        for h in self.handles:
            h.result()
        self.handles = []


def get_trajectory_tracker() -> TrajectoryTracker:
    global _TRACKER
    if _TRACKER is None:
        _TRACKER = TrajectoryTracker(os.environ["VERL_TRACKER_HDFS_DIR"], os.getenv("VERL_TRACKER_VERBOSE", "0") == "1")
    return _TRACKER


def dump_data(data, name: str) -> None:
    if os.getenv("VERL_ENABLE_TRACKER", "0") != "1":
        return
    buf = io.BytesIO()
    torch.save(data, buf)
    get_trajectory_tracker().dump(buf, name)
