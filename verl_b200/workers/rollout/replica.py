"""Rollout replicas: one inference endpoint spanning TP x DP x PP GPUs (verl/workers/rollout/replica.py:32-339).

Modes: HYBRID (shares processes and GPUs with trainer workers), COLOCATED (same GPUs, own processes),
STANDALONE (own GPUs). On one box every mode is served by the native engine; a replica exposes the server
handle(s) that the agent loop's load balancer talks to.
"""

from __future__ import annotations

import asyncio
from abc import ABC
from enum import Enum
from typing import Any, Callable, Optional

from ...rollout import TokenOutput  # noqa: F401  (re-exported: the reference defines it here)


class RolloutMode(Enum):
    HYBRID = "hybrid"
    COLOCATED = "colocated"
    STANDALONE = "standalone"


class RolloutReplica(ABC):
    def __init__(self, replica_rank: int, config, model_config, gpus_per_node: int = 8, is_reward_model: bool = False):
        self.replica_rank = replica_rank
        self.config, self.model_config = config, model_config
        g = (lambda k, d=1: int(getattr(config, k, d) or d)) if not isinstance(config, dict) else (lambda k, d=1: int(config.get(k, d) or d))
        self.world_size = g("tensor_model_parallel_size") * g("data_parallel_size") * g("pipeline_model_parallel_size")
        self.gpus_per_node = min(gpus_per_node, self.world_size)
        assert self.world_size % self.gpus_per_node == 0
        self.nnodes = self.world_size // self.gpus_per_node
        self.is_reward_model = is_reward_model
        self.rollout_mode: Optional[RolloutMode] = None
        self.workers: list = []
        self.resource_pool = None
        self.servers: list = []
        self._server_address = None
        self._server_handle = None

    async def init_hybrid(self, worker_group):
        """Serve from the trainer's own worker processes (ranks [r*ws, (r+1)*ws) of the worker group)."""
        self.rollout_mode = RolloutMode.HYBRID
        ws = self.world_size
        self.workers = list(getattr(worker_group, "workers", []))[ws * self.replica_rank : ws * (self.replica_rank + 1)]
        await self.launch_servers()

    async def init_hybrid_colocated(self, worker_group, resource_pool):
        """The trainer's worker processes serve (as in :meth:`init_hybrid`) and the replica remembers the resource pool
        those processes live in, for helpers that are placed beside them."""
        self.resource_pool = resource_pool
        await self.init_hybrid(worker_group)
        self.rollout_mode = RolloutMode.HYBRID

    def get_ray_class_with_init_args(self):
        """Worker class (+ constructor arguments) of a replica that starts its own processes (COLOCATED / STANDALONE)."""
        raise NotImplementedError

    def rollout_worker_use_gpu(self) -> bool:
        return True

    async def init_colocated(self, resource_pool):
        self.rollout_mode = RolloutMode.COLOCATED
        self.resource_pool = resource_pool
        await self.launch_servers()

    async def init_standalone(self):
        self.rollout_mode = RolloutMode.STANDALONE
        await self.launch_servers()

    async def launch_servers(self):
        raise NotImplementedError

    @property
    def server_address(self) -> Optional[str]:
        return self._server_address

    @property
    def server_handle(self):
        return self._server_handle

    async def wake_up(self):
        await asyncio.gather(*[s.wake_up() for s in self.servers])

    async def sleep(self):
        await asyncio.gather(*[s.sleep() for s in self.servers])

    async def abort_all_requests(self):
        res = await asyncio.gather(*[s.abort_all_requests() for s in self.servers])
        return {"aborted_count": sum(r["aborted_count"] for r in res), "request_ids": sum((r["request_ids"] for r in res), [])}

    async def resume_all_requests(self):
        await asyncio.gather(*[s.resume_all_requests() for s in self.servers])

    async def clear_kv_cache(self):
        await asyncio.gather(*[s.clear_kv_cache() for s in self.servers])

    async def start_profile(self, **kwargs):
        await asyncio.gather(*[s.start_profile(**kwargs) for s in self.servers])

    async def stop_profile(self):
        await asyncio.gather(*[s.stop_profile() for s in self.servers])


class NativeReplica(RolloutReplica):
    """Replica backed by in-process native engines. ``engine_factory()`` builds the engine in STANDALONE /
    COLOCATED mode; in HYBRID mode ``engine`` is the trainer worker's engine."""

    def __init__(self, replica_rank, config, model_config, gpus_per_node: int = 8, is_reward_model: bool = False,
                 engine=None, engine_factory: Optional[Callable] = None):
        super().__init__(replica_rank, config, model_config, gpus_per_node, is_reward_model)
        self._engine, self._factory = engine, engine_factory

    async def launch_servers(self):
        from .async_server import NativeAsyncServer

        eng = self._engine if self._engine is not None else self._factory()
        g = (lambda k, d: getattr(self.config, k, d)) if not isinstance(self.config, dict) else (lambda k, d: self.config.get(k, d))
        srv = NativeAsyncServer(eng, response_length=int(g("response_length", 512)), prompt_length=int(g("prompt_length", 512)))
        self.servers = [srv]
        self._server_handle = srv
        self._server_address = f"inproc://replica-{self.replica_rank}"


class RolloutReplicaRegistry:
    _registry: dict[str, Callable[[], type]] = {}

    @classmethod
    def register(cls, name: str, loader: Callable[[], type]) -> None:
        cls._registry[name] = loader

    @classmethod
    def get(cls, name: str) -> type[RolloutReplica]:
        if name not in cls._registry:
            raise ValueError(f"Unknown rollout mode: {name}. Supported: {list(cls._registry.keys())}")
        return cls._registry[name]()


for _name in ("native", "vllm", "sglang", "trtllm"):
    RolloutReplicaRegistry.register(_name, lambda: NativeReplica)


def get_rollout_replica_class(rollout: str) -> type[RolloutReplica]:
    return RolloutReplicaRegistry.get(rollout)
