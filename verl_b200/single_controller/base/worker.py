"""Base class of SPMD workers (one process per GPU / per CPU rank).

Counterpart of verl/single_controller/base/worker.py:76-357: reads its rank from the environment
set by the worker group (``WORLD_SIZE, RANK, LOCAL_WORLD_SIZE, LOCAL_RANK, MASTER_ADDR,
MASTER_PORT``), records (mesh_name -> dp_rank, is_collect) for mesh-aware dispatch, and offers
``execute_with_func_generator`` / ``execute_func_rank_zero`` for ad-hoc remote functions.
"""

from __future__ import annotations

import os
import socket
from dataclasses import dataclass

from .decorator import Dispatch, Execute, register


@dataclass
class DistRankInfo:
    tp_rank: int
    dp_rank: int
    pp_rank: int
    cp_rank: int


@dataclass
class DistGlobalInfo:
    tp_size: int
    dp_size: int
    pp_size: int
    cp_size: int


class WorkerHelper:
    @staticmethod
    def _get_node_ip() -> str:
        try:
            return socket.gethostbyname(socket.gethostname())
        except OSError:
            return "127.0.0.1"

    @staticmethod
    def _get_free_port() -> int:
        with socket.socket() as s:
            s.bind(("", 0))
            return s.getsockname()[1]

    def get_availale_master_addr_port(self):
        return self._get_node_ip(), str(self._get_free_port())


class Worker(WorkerHelper):
    """A remotely-driven worker. Subclasses add ``@register``-decorated methods."""

    fused_worker_attr_name = "fused_worker_dict"

    def __new__(cls, *args, **kwargs):
        inst = super().__new__(cls)
        inst.__dispatch_dp_rank = {}
        inst.__collect_dp_rank = {}
        return inst

    def __init__(self, cuda_visible_devices=None) -> None:
        env = os.environ
        self._world_size = int(env.get("WORLD_SIZE", 1))
        self._rank = int(env.get("RANK", 0))
        self._local_world_size = int(env.get("LOCAL_WORLD_SIZE", self._world_size))
        self._local_rank = int(env.get("LOCAL_RANK", self._rank))
        self._master_addr = env.get("MASTER_ADDR", "127.0.0.1")
        self._master_port = env.get("MASTER_PORT", "29500")
        self._cuda_visible_devices = cuda_visible_devices or env.get("CUDA_VISIBLE_DEVICES")
        self.fused_worker_dict = {}
        if not hasattr(self, "_Worker__dispatch_dp_rank"):
            self.__dispatch_dp_rank, self.__collect_dp_rank = {}, {}

    # ---- mesh-aware dispatch bookkeeping --------------------------------------
    def _register_dispatch_collect_info(self, mesh_name: str, dp_rank: int, is_collect: bool):
        if mesh_name in self.__dispatch_dp_rank:
            raise ValueError(f"mesh_name {mesh_name} has been registered")
        self.__dispatch_dp_rank[mesh_name] = dp_rank
        self.__collect_dp_rank[mesh_name] = is_collect

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def _query_dispatch_info(self, mesh_name: str):
        assert mesh_name in self.__dispatch_dp_rank, f"{mesh_name} is not registered in {self.__class__.__name__}"
        return self.__dispatch_dp_rank[mesh_name]

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def _query_collect_info(self, mesh_name: str):
        assert mesh_name in self.__collect_dp_rank, f"{mesh_name} is not registered in {self.__class__.__name__}"
        return self.__collect_dp_rank[mesh_name]

    def query_collect_info(self, mesh_name: str) -> bool:
        """Whether this worker's output is collected for ``mesh_name`` (plain method: for callers inside the worker)."""
        assert mesh_name in self.__collect_dp_rank, f"{mesh_name} is not registered in {self.__class__.__name__}"
        return self.__collect_dp_rank[mesh_name]

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def get_dispatch_collect(self) -> dict:
        """All registered meshes: ``{"dispatch_dp_rank": {mesh: dp rank}, "collect_dp_rank": {mesh: bool}}``."""
        return {"dispatch_dp_rank": dict(self.__dispatch_dp_rank), "collect_dp_rank": dict(self.__collect_dp_rank)}

    @register(dispatch_mode=Dispatch.ALL_TO_ALL)
    def set_dispatch_collect(self, mesh_name: str, dispatch_dp_rank: dict, collect_dp_rank: dict) -> None:
        """Give ``mesh_name`` the registration of another mesh's layout on this worker: the dictionaries are those of
        :meth:`get_dispatch_collect` of the worker that should be mirrored (a role that shares another role's
        data-parallel layout without building an engine of its own)."""
        assert mesh_name not in self.__dispatch_dp_rank, f"{mesh_name} is already registered"
        src = next(iter(dispatch_dp_rank)) if len(dispatch_dp_rank) == 1 else mesh_name
        self.__dispatch_dp_rank[mesh_name] = dispatch_dp_rank[src]
        self.__collect_dp_rank[mesh_name] = collect_dp_rank[src]

    def get_fused_worker_by_name(self, worker_name: str):
        return self.fused_worker_dict.get(worker_name, None)

    # ---- environment ------------------------------------------------------------
    @property
    def world_size(self) -> int:
        return self._world_size

    @property
    def rank(self) -> int:
        return self._rank

    @property
    def local_rank(self) -> int:
        return self._local_rank

    def get_master_addr_port(self):
        return self._master_addr, self._master_port

    def get_cuda_visible_devices(self):
        return os.environ.get("CUDA_VISIBLE_DEVICES", "not set")

    @classmethod
    def env_keys(cls):
        return ["WORLD_SIZE", "RANK", "LOCAL_WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT",
                "CUDA_VISIBLE_DEVICES"]

    # ---- generic remote execution -----------------------------------------------
    @register(dispatch_mode=Dispatch.DP_COMPUTE_PROTO_WITH_FUNC)
    def execute_with_func_generator(self, func, *args, **kwargs):
        return func(self, *args, **kwargs)

    @register(dispatch_mode=Dispatch.ALL_TO_ALL, execute_mode=Execute.RANK_ZERO)
    def execute_func_rank_zero(self, func, *args, **kwargs):
        return func(*args, **kwargs)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def ping(self):
        return self._rank
