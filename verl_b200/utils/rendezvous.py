"""Rendezvous of a side communicator by NAME between processes that share no process group yet (role of
verl/utils/rendezvous/ray_backend.py:24-73, where rank 0 parks an NCCL unique id in a named Ray actor and the other
ranks look the actor up with retries). Here rank 0 opens a TCP store on a free port and publishes ``host:port`` as a
small file named after the group in a registry directory that all ranks can read (one box: ``/dev/shm`` or the
temporary directory; several boxes: a shared file system); the others poll for it and all ranks build a process group
on that store (NCCL on CUDA devices, gloo otherwise), independent of the default group."""

from __future__ import annotations

import json
import os
import tempfile
import time
from typing import Optional

import torch.distributed as dist

from .distributed import stateless_init_process_group
from .net_utils import get_free_port


def _registry(registry_dir: Optional[str]) -> str:
    d = registry_dir or os.environ.get("VERL_B200_RENDEZVOUS_DIR") or os.path.join(tempfile.gettempdir(), "verl_b200_rendezvous")
    os.makedirs(d, exist_ok=True)
    return d


def publish_endpoint(group_name: str, host: str, port: int, registry_dir: Optional[str] = None) -> str:
    path = os.path.join(_registry(registry_dir), f"{group_name}.json")
    tmp = f"{path}.{os.getpid()}.tmp"
    with open(tmp, "w") as f:
        json.dump({"host": host, "port": int(port), "pid": os.getpid(), "time": time.time()}, f)
    os.replace(tmp, path)  # atomic: a reader sees the whole record or none
    return path


def lookup_endpoint(group_name: str, registry_dir: Optional[str] = None, max_retries: int = 100,
                    interval_s: float = 0.2) -> Optional[dict]:
    path = os.path.join(_registry(registry_dir), f"{group_name}.json")
    for _ in range(max(1, max_retries)):
        try:
            with open(path) as f:
                return json.load(f)
        except (FileNotFoundError, json.JSONDecodeError):
            time.sleep(interval_s)
    return None


def create_communicator_by_name(rank: int, world_size: int, group_name: str, device=None, host: str = "127.0.0.1",
                                registry_dir: Optional[str] = None, max_retries: int = 100, interval_s: float = 0.2,
                                timeout_s: int = 600) -> dist.ProcessGroup:
    """Every rank calls this with the same ``group_name``; returns a process group of ``world_size`` ranks."""
    if rank == 0:
        port = get_free_port(host)
        path = publish_endpoint(group_name, host, port, registry_dir)
        try:
            return stateless_init_process_group(host, port, 0, world_size, device=device, timeout_s=timeout_s)
        finally:
            try:
                os.remove(path)  # every rank has connected by now: the name can be used again
            except FileNotFoundError:
                pass
    ep = lookup_endpoint(group_name, registry_dir, max_retries, interval_s)
    if ep is None:
        raise TimeoutError(f"no endpoint was published for communicator {group_name!r} within "
                           f"{max_retries * interval_s:.0f} s")
    return stateless_init_process_group(ep["host"], ep["port"], rank, world_size, device=device, timeout_s=timeout_s)
