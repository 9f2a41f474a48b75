"""Weight sync through pinned host buckets with an overlap thread (the engine of the fully asynchronous pipeline).

Role of verl/experimental/fully_async_policy/checkpoint_engine.py:259-520: the trainer registers its weights once;
every trainer rank owns a share of fixed buckets in pinned host memory and refreshes them after an update
(device -> pinned host, on a side stream, so the next training step does not wait); a sync then streams the buckets
host -> device -> (broadcast) -> consumer with two device buffers, the transfer of bucket i + 1 running on a thread
while the rollout engine consumes bucket i.

Differences by design: the staging copies are issued as ONE flat copy per bucket out of a packed device scratch when
the source tensors are on a CUDA device (a copy per tensor would be launch-bound for thousands of small tensors); a
bucket never splits a tensor; offsets are 256-byte aligned so that every view satisfies the alignment of the kernels
that read it.
"""

from __future__ import annotations

import queue
import threading
from dataclasses import dataclass, field
from typing import Callable, Iterable, Optional

import torch

from .base import CheckpointEngine, CheckpointEngineRegistry, TensorMeta

_ALIGN = 256


def _nbytes(shape, dtype) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n * torch.empty(0, dtype=dtype).element_size()


@dataclass
class Bucket:
    owner: int                      # trainer rank that stages and sends this bucket
    nbytes: int = 0
    metas: list = field(default_factory=list)  # TensorMeta with offsets inside the bucket


def plan_buckets(weights_info: Iterable[tuple[str, tuple, torch.dtype]], bucket_bytes: int, num_owners: int = 1) -> list[Bucket]:
    """Greedy packing in registration order; a tensor larger than ``bucket_bytes`` gets a bucket of its own. Buckets
    are dealt to the owners round-robin, so every trainer rank sends about the same number of bytes."""
    buckets: list[Bucket] = []
    cur = Bucket(owner=0)
    for name, shape, dtype in weights_info:
        nb = _nbytes(shape, dtype)
        if cur.metas and cur.nbytes + nb > bucket_bytes:
            buckets.append(cur)
            cur = Bucket(owner=0)
        cur.metas.append(TensorMeta(name, tuple(shape), dtype, cur.nbytes))
        cur.nbytes = (cur.nbytes + nb + _ALIGN - 1) // _ALIGN * _ALIGN
    if cur.metas:
        buckets.append(cur)
    for i, b in enumerate(buckets):
        b.owner = i % max(num_owners, 1)
    return buckets


def views_of(bucket: Bucket, buf: torch.Tensor) -> list[tuple[str, torch.Tensor]]:
    out = []
    for m in bucket.metas:
        nb = _nbytes(m.shape, m.dtype)
        out.append((m.name, buf[m.offset : m.offset + nb].view(m.dtype).view(m.shape)))
    return out


@CheckpointEngineRegistry.register("pinned_async")
class PinnedBucketEngine(CheckpointEngine):
    """``register`` once, ``stage`` after every optimizer step (asynchronous), ``publish`` when the rollout side takes
    the new version.

    ``rank`` / ``trainer_ranks`` / ``group``: with a process group every bucket is broadcast from its owner to all
    ranks of the group (trainer and rollout ranks alike); without one the engine serves a consumer in the same
    process. ``device``: where the consumer wants its tensors."""

    def __init__(self, bucket_size: int = 512 << 20, rank: int = 0, trainer_ranks: Optional[list[int]] = None, group=None,
                 device=None, **kwargs):
        self.bucket_size = int(bucket_size)
        self.rank = int(rank)
        self.trainer_ranks = list(trainer_ranks) if trainer_ranks is not None else [self.rank]
        self.group = group
        self.device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self.buckets: list[Bucket] = []
        self.host: dict[int, torch.Tensor] = {}   # bucket index -> pinned host buffer (owned buckets only)
        self._stage_event = None
        self._stage_stream = None
        self.version = -1
        self.stats = {"staged_bytes": 0, "published_bytes": 0, "buckets": 0}

    # ------------------------------------------------------------------ CheckpointEngine interface
    def prepare(self):
        return {"bucket_size": self.bucket_size, "buckets": len(self.buckets)}

    @classmethod
    def build_topology(cls, trainer_world_size, rollout_world_size, metadata):
        w = trainer_world_size + rollout_world_size
        return ({"rank": list(range(trainer_world_size)), "world_size": [w] * trainer_world_size},
                {"rank": list(range(trainer_world_size, w)), "world_size": [w] * rollout_world_size})

    def init_process_group(self, group=None, **kwargs):
        if group is not None:
            self.group = group

    def finalize(self):
        self.wait_staged()
        self.host.clear()
        self.buckets = []

    async def send_weights(self, weights):
        named = list(weights)
        if not self.buckets:
            self.register([(n, tuple(t.shape), t.dtype) for n, t in named])
        self.stage(dict(named))
        self.publish(lambda pairs: None)

    async def receive_weights(self):
        got: list = []
        self.publish(lambda pairs: got.extend((n, t.clone()) for n, t in pairs))
        for item in got:
            yield item

    # ------------------------------------------------------------------ registration and staging (trainer side)
    def register(self, weights_info: Iterable[tuple[str, tuple, torch.dtype]]):
        """Fix the bucket layout (every rank computes the same one) and pin the host memory of the owned buckets."""
        self.buckets = plan_buckets(weights_info, self.bucket_size, len(self.trainer_ranks))
        pin = torch.cuda.is_available()
        self.host = {}
        for i, b in enumerate(self.buckets):
            if self.trainer_ranks[b.owner] == self.rank:
                self.host[i] = torch.empty(b.nbytes, dtype=torch.uint8, pin_memory=pin)
        self.stats["buckets"] = len(self.buckets)
        return self.buckets

    def stage(self, named_tensors: dict, version: Optional[int] = None):
        """Refresh the owned pinned buckets from the current weights. On CUDA the copies run on a side stream that
        first waits for the calling stream (so it sees the finished optimizer step); the call returns at once and
        ``wait_staged`` / ``publish`` wait for the copies."""
        assert self.buckets, "register() first"
        on_cuda = any(t.is_cuda for t in named_tensors.values())
        if on_cuda:
            if self._stage_stream is None:
                self._stage_stream = torch.cuda.Stream()
            self._stage_stream.wait_stream(torch.cuda.current_stream())
        ctx = torch.cuda.stream(self._stage_stream) if on_cuda else _null()
        staged = 0
        with ctx, torch.no_grad():
            for i, buf in self.host.items():
                b = self.buckets[i]
                if on_cuda:
                    # pack on the device, then ONE device -> host copy per bucket
                    scratch = torch.empty(b.nbytes, dtype=torch.uint8, device=next(iter(named_tensors.values())).device)
                    for name, view in views_of(b, scratch):
                        view.copy_(named_tensors[name])
                    buf.copy_(scratch, non_blocking=True)
                    scratch.record_stream(self._stage_stream)
                else:
                    for name, view in views_of(b, buf):
                        view.copy_(named_tensors[name])
                staged += b.nbytes
            if on_cuda:
                self._stage_event = torch.cuda.Event()
                self._stage_event.record(self._stage_stream)
        self.stats["staged_bytes"] += staged
        if version is not None:
            self.version = int(version)

    def wait_staged(self):
        if self._stage_event is not None:
            self._stage_event.synchronize()
            self._stage_event = None

    # ------------------------------------------------------------------ publishing (all ranks)
    def publish(self, consume: Callable[[list[tuple[str, torch.Tensor]]], None], depth: int = 2):
        """Stream every bucket to ``consume`` as (name, tensor-on-device) pairs. A producer thread moves bucket i + 1
        (host -> device, then the broadcast when there is a group) into one of ``depth`` device buffers while
        ``consume`` works on bucket i; a buffer is reused only after its consumer has returned."""
        assert self.buckets, "register() first"
        self.wait_staged()
        cap = max(b.nbytes for b in self.buckets)
        bufs = [torch.empty(cap, dtype=torch.uint8, device=self.device) for _ in range(depth)]
        free: queue.Queue = queue.Queue()
        ready: queue.Queue = queue.Queue()
        for k in range(depth):
            free.put(k)
        err: list = []
        use_cuda = self.device.type == "cuda"
        copy_stream = torch.cuda.Stream(device=self.device) if use_cuda else None

        def producer():
            try:
                if use_cuda:
                    torch.cuda.set_device(self.device)
                for i, b in enumerate(self.buckets):
                    k = free.get()
                    if stop.is_set():
                        break
                    dst = bufs[k][: b.nbytes]
                    ctx = torch.cuda.stream(copy_stream) if use_cuda else _null()
                    with ctx:
                        if i in self.host:
                            dst.copy_(self.host[i], non_blocking=True)
                        if self.group is not None:
                            import torch.distributed as dist

                            dist.broadcast(dst, src=dist.get_global_rank(self.group, self._group_index(b.owner)), group=self.group)
                        ev = None
                        if use_cuda:
                            ev = torch.cuda.Event()
                            ev.record(copy_stream)
                    ready.put((i, k, ev))
            except BaseException as e:  # hand the failure to the consuming thread
                err.append(e)
            finally:
                ready.put(None)

        stop = threading.Event()
        th = threading.Thread(target=producer, name="pinned-bucket-producer", daemon=True)
        th.start()
        done = 0
        try:
            while True:
                item = ready.get()
                if item is None:
                    break
                i, k, ev = item
                if ev is not None:
                    torch.cuda.current_stream(self.device).wait_event(ev)
                consume(views_of(self.buckets[i], bufs[k]))
                if use_cuda:
                    torch.cuda.current_stream(self.device).synchronize()  # the buffer goes back when its readers are done
                free.put(k)
                done += self.buckets[i].nbytes
        except BaseException:
            stop.set()  # a failing consumer must not leave the producer waiting for a buffer
            for k in range(depth):
                free.put(k)
            th.join()
            raise
        th.join()
        if err:
            raise err[0]
        self.stats["published_bytes"] += done
        return done

    def _group_index(self, owner: int) -> int:
        """Rank inside ``group`` of the trainer rank that owns a bucket (the group lists trainer ranks first)."""
        import torch.distributed as dist

        ranks = dist.get_process_group_ranks(self.group)
        return ranks.index(self.trainer_ranks[owner])


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
