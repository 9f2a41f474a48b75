"""Process-group bootstrap helpers (role of verl/utils/distributed.py:27-165)."""

from __future__ import annotations

import ctypes
import datetime
import os
from typing import Optional

import torch
import torch.distributed as dist

from .device import get_nccl_backend


def set_numa_affinity() -> None:
    """Bind the process to the NUMA node of its GPU when libnuma and NVML are there (best effort, silent otherwise)."""
    try:
        import pynvml

        libnuma = ctypes.CDLL("libnuma.so.1")
        if libnuma.numa_available() < 0:
            return
        pynvml.nvmlInit()
        idx = int(os.environ.get("LOCAL_RANK", "0"))
        handle = pynvml.nvmlDeviceGetHandleByIndex(idx)
        node = pynvml.nvmlDeviceGetNumaNodeId(handle) if hasattr(pynvml, "nvmlDeviceGetNumaNodeId") else -1
        if node >= 0:
            libnuma.numa_run_on_node(ctypes.c_int(node))
            libnuma.numa_set_preferred(ctypes.c_int(node))
    except Exception:
        return


def initialize_global_process_group(timeout_second: int = 36000):
    """torchrun-style init from RANK / LOCAL_RANK / WORLD_SIZE; returns (local_rank, rank, world_size)."""
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    backend = get_nccl_backend()
    if not dist.is_initialized():
        dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_second))
    local_rank, rank, world = int(os.environ.get("LOCAL_RANK", 0)), dist.get_rank(), dist.get_world_size()
    if torch.cuda.is_available():
        torch.cuda.set_device(local_rank)
    return local_rank, rank, world


def destroy_global_process_group() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()


def stateless_init_process_group(master_address: str, master_port: int, rank: int, world_size: int, device=None,
                                 timeout_s: int = 600) -> dist.ProcessGroup:
    """A process group that is independent of the default one (trainer <-> rollout weight-sync groups between
    otherwise unrelated jobs; the reference builds this from vLLM's StatelessProcessGroup + PyNcclCommunicator,
    verl/utils/distributed.py:83-165). Here: a TCPStore rendezvous and a torch ProcessGroup on top of it."""
    store = dist.TCPStore(master_address, int(master_port), world_size, is_master=(rank == 0),
                          timeout=datetime.timedelta(seconds=timeout_s))
    backend = "nccl" if (device is not None and torch.device(device).type == "cuda") else "gloo"
    prefix = dist.PrefixStore(f"stateless_{master_port}", store)
    if backend == "gloo":
        pg = dist.ProcessGroupGloo(prefix, rank, world_size, datetime.timedelta(seconds=timeout_s))
    else:
        opts = dist.ProcessGroupNCCL.Options()
        pg = dist.ProcessGroupNCCL(prefix, rank, world_size, opts)
    return pg


def initialize_global_process_group_ray(timeout_second: Optional[int] = None, backend: Optional[str] = None) -> None:
    """Default process group of a worker that a controller started with RANK / WORLD_SIZE / MASTER_* in its environment
    (the worker groups of this framework set them); ``backend`` such as ``"cpu:gloo,cuda:nccl"`` or ``"cpu:gloo"``."""
    if dist.is_initialized():
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    kw = {"timeout": datetime.timedelta(seconds=timeout_second)} if timeout_second is not None else {}
    dist.init_process_group(backend=backend or get_nccl_backend(), rank=int(os.environ.get("RANK", 0)),
                            world_size=int(os.environ.get("WORLD_SIZE", 1)), **kw)
