"""Weight synchronisation ("checkpoint engine") between trainer and rollout replicas.

Abstractions of verl/checkpoint_engine/base.py:30-410: ``TensorMeta``, ``CheckpointEngineRegistry``, the
``CheckpointEngine`` protocol (``prepare / build_topology / init_process_group / finalize / send_weights /
receive_weights``), ``ColocatedCheckpointEngine`` ("naive": trainer hands a generator to the colocated rollout),
and ``CheckpointEngineManager`` orchestrating a sync across trainer workers and replicas (abort in-flight
requests -> sync -> resume).

Backends here: ``naive`` (colocated generator), ``nvlink`` (single-kernel reshard over peer memory,
:mod:`verl_b200.parallel.reshard`), ``nccl`` (bucketed broadcast through torch.distributed for replicas that are
separate processes).
"""

from __future__ import annotations

import asyncio
from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any, Generator, Optional

import torch


@dataclass
class TensorMeta:
    name: str
    shape: torch.Size
    dtype: torch.dtype
    offset: int


class CheckpointEngineRegistry:
    _registry: dict[str, type["CheckpointEngine"]] = {}

    @classmethod
    def register(cls, backend: str):
        def deco(engine_cls):
            cls._registry[backend] = engine_cls
            return engine_cls

        return deco

    @classmethod
    def get(cls, backend: str) -> type["CheckpointEngine"]:
        if backend not in cls._registry:
            raise ValueError(f"Unknown checkpoint engine backend: {backend}. Available: {list(cls._registry)}")
        return cls._registry[backend]

    @classmethod
    def new(cls, backend: str, *args, **kwargs) -> "CheckpointEngine":
        return cls.get(backend)(*args, **kwargs)


def build_checkpoint_engine(config, **kwargs) -> "CheckpointEngine":
    """Engine of ``rollout.checkpoint_engine`` (``backend``, ``update_weights_bucket_megabytes``,
    ``engine_kwargs[backend]``); ``kwargs`` are the call site's own arguments (process group, role, device)."""
    get = config.get if hasattr(config, "get") else (lambda k, d=None: getattr(config, k, d))
    backend = get("backend", "naive") or "naive"
    extra = dict((get("engine_kwargs", None) or {}).get(backend, None) or {})
    mb = int(get("update_weights_bucket_megabytes", 2048) or 2048)
    return CheckpointEngineRegistry.new(backend, **{"bucket_size": mb << 20, **extra, **kwargs})


class CheckpointEngine(ABC):
    """One side (trainer or rollout) of a weight transfer."""

    @abstractmethod
    def prepare(self) -> Any:
        """Allocate buffers; returns metadata the manager exchanges to build the topology."""

    @classmethod
    @abstractmethod
    def build_topology(cls, trainer_world_size: int, rollout_world_size: int, metadata: list) -> tuple[dict, dict]:
        """Per-rank kwargs for ``init_process_group`` of trainer and rollout workers."""

    @abstractmethod
    def init_process_group(self, **kwargs):
        ...

    @abstractmethod
    def finalize(self):
        ...

    @abstractmethod
    async def send_weights(self, weights: Generator[tuple[str, torch.Tensor], None, None]):
        ...

    @abstractmethod
    async def receive_weights(self) -> Generator[tuple[str, torch.Tensor], None, None]:
        ...


class CheckpointEngineWithCache(CheckpointEngine):
    """Keeps the last received weights so replicas that join later can be served without the trainer."""

    def __init__(self):
        self._cache: dict[str, torch.Tensor] = {}

    def cache(self, name: str, t: torch.Tensor):
        self._cache[name] = t.detach().cpu()

    def cached_weights(self):
        yield from self._cache.items()


@CheckpointEngineRegistry.register("naive")
class ColocatedCheckpointEngine(CheckpointEngine):
    """Trainer and rollout share the process: ``send_weights`` stores the generator, ``receive_weights`` drains it."""

    def __init__(self, bucket_size: int = 2048 << 20, **kwargs):
        self.bucket_size = bucket_size
        self._weights = None

    def prepare(self):
        return None

    @classmethod
    def build_topology(cls, trainer_world_size, rollout_world_size, metadata):
        return {"rank": list(range(trainer_world_size))}, {"rank": list(range(rollout_world_size))}

    def init_process_group(self, **kwargs):
        pass

    def finalize(self):
        self._weights = None

    async def send_weights(self, weights):
        self._weights = weights

    async def receive_weights(self):
        assert self._weights is not None, "send_weights() must be called first"
        for item in self._weights:
            yield item
        self._weights = None


@CheckpointEngineRegistry.register("nvlink")
class NVLinkCheckpointEngine(ColocatedCheckpointEngine):
    """Hybrid workers on one NVSwitch domain: the sync is ``RolloutWeights.sync()`` — one kernel that pulls every
    peer's ZeRO shard into this rank's rollout layout. The generator protocol is kept for API parity; the fast path
    is taken by ``ActorRolloutRefWorker.update_weights``."""


@CheckpointEngineRegistry.register("nccl")
class NCCLCheckpointEngine(CheckpointEngineWithCache):
    """Bucketed broadcast from trainer rank 0 to rollout ranks over a torch.distributed group (role of
    verl/checkpoint_engine/nccl_checkpoint_engine.py:97-363 for replicas in other processes). Two buckets alternate
    so packing the next bucket overlaps the broadcast of the current one."""

    def __init__(self, bucket_size: int = 2048 << 20, group=None, is_master: bool = False, src: int = 0, device=None, **kw):
        super().__init__()
        self.bucket_size, self.group, self.is_master, self.src = bucket_size, group, is_master, src
        self.device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self._buckets = None

    def prepare(self):
        self._buckets = [torch.empty(self.bucket_size, dtype=torch.uint8, device=self.device) for _ in range(2)]
        return {"bucket_size": self.bucket_size}

    @classmethod
    def build_topology(cls, trainer_world_size, rollout_world_size, metadata):
        tr = {"rank": [0] + [-1] * (trainer_world_size - 1), "world_size": [rollout_world_size + 1] * trainer_world_size}
        ro = {"rank": list(range(1, rollout_world_size + 1)), "world_size": [rollout_world_size + 1] * rollout_world_size}
        return tr, ro

    def init_process_group(self, group=None, **kwargs):
        if group is not None:
            self.group = group

    def finalize(self):
        self._buckets = None

    def _bcast_obj(self, obj):
        import torch.distributed as dist

        box = [obj]
        dist.broadcast_object_list(box, src=self.src, group=self.group)
        return box[0]

    async def send_weights(self, weights):
        import torch.distributed as dist

        if self._buckets is None:
            self.prepare()
        which, off, metas = 0, 0, []

        def flush(last: bool):
            nonlocal which, off, metas
            self._bcast_obj({"metas": metas, "nbytes": off, "last": last})
            if off:
                dist.broadcast(self._buckets[which][:off], src=self.src, group=self.group)
            which, off, metas = which ^ 1, 0, []

        for name, t in weights:
            t = t.detach().contiguous()
            nbytes = t.numel() * t.element_size()
            assert nbytes <= self.bucket_size, f"{name} ({nbytes} B) exceeds the bucket size {self.bucket_size}"
            if off + nbytes > self.bucket_size:
                flush(False)
            self._buckets[which][off : off + nbytes].copy_(t.view(torch.uint8).reshape(-1))
            metas.append(TensorMeta(name, t.shape, t.dtype, off))
            off += (nbytes + 255) // 256 * 256
        flush(True)

    async def receive_weights(self):
        import torch.distributed as dist

        if self._buckets is None:
            self.prepare()
        which = 0
        while True:
            head = self._bcast_obj(None)
            if head["nbytes"]:
                dist.broadcast(self._buckets[which][: head["nbytes"]], src=self.src, group=self.group)
            for m in head["metas"]:
                n = int(torch.tensor(m.shape).prod()) * torch.empty(0, dtype=m.dtype).element_size() if len(m.shape) else torch.empty(0, dtype=m.dtype).element_size()
                t = self._buckets[which][m.offset : m.offset + n].view(m.dtype).view(m.shape)
                yield m.name, t
            which ^= 1
            if head["last"]:
                break


class CheckpointEngineWorker:
    """The rollout side of a weight transfer as a worker: owns a checkpoint engine built from
    ``rollout.checkpoint_engine`` and a rollout adapter (anything with ``update_weights(iterator of (name, tensor))``);
    ``update_weights`` receives what the trainer side sends and hands it to the adapter
    (verl/checkpoint_engine/base.py:244-280). Worker groups call its two methods on every replica process."""

    def __init__(self, rollout_config, model_config=None, server_adapter=None, **engine_kwargs):
        self.rollout_config, self.model_config, self.server_adapter = rollout_config, model_config, server_adapter
        get = rollout_config.get if hasattr(rollout_config, "get") else (lambda k, d=None: getattr(rollout_config, k, d))
        self.checkpoint_engine = build_checkpoint_engine(get("checkpoint_engine", None) or {}, **engine_kwargs)

    async def update_weights(self):
        async def feed(items):
            res = self.server_adapter.update_weights(items)
            if asyncio.iscoroutine(res):
                await res

        weights = self.checkpoint_engine.receive_weights()
        if hasattr(weights, "__aiter__"):
            # tensors are views of a bucket that the next bucket overwrites: the adapter takes each one as it arrives
            async for item in weights:
                await feed(iter([item]))
        else:
            await feed(weights)

    def execute_checkpoint_engine(self, method: str, *args, **kwargs):
        return getattr(self.checkpoint_engine, method)(*args, **kwargs)


class CheckpointEngineManager:
    """Drives a weight sync: trainer worker group -> rollout replicas (verl/checkpoint_engine/base.py:286-410)."""

    def __init__(self, backend: str, trainer, replicas: Optional[list] = None):
        self.backend = backend
        self.trainer = trainer
        self.replicas = list(replicas or [])

    def add_replicas(self, replicas: list):
        self.replicas.extend(replicas)

    def remove_replicas(self, replicas: list):
        self.replicas = [r for r in self.replicas if r not in replicas]

    def sleep_replicas(self):
        async def go():
            await asyncio.gather(*[r.sleep() for r in self.replicas])

        if self.replicas:
            asyncio.run(go())

    def update_weights(self, global_steps: Optional[int] = None):
        """Colocated backends: one RPC to the hybrid workers. Replica processes: abort -> sync -> resume."""
        async def pre():
            await asyncio.gather(*[r.abort_all_requests() for r in self.replicas])

        async def post():
            await asyncio.gather(*[r.resume_all_requests() for r in self.replicas])

        if self.replicas and self.backend not in ("naive", "nvlink"):
            asyncio.run(pre())
        res = self.trainer.update_weights(global_steps)
        res = res.result() if hasattr(res, "result") else res
        if isinstance(res, (list, tuple)):  # one future per worker: wait for every one before the replicas resume
            res = [r.result() if hasattr(r, "result") else r for r in res]
            res = res[0] if res else None
        if self.replicas and self.backend not in ("naive", "nvlink"):
            asyncio.run(post())
        return res
