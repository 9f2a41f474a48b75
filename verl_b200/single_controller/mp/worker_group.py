"""Multiprocess single-controller backend: one OS process per rank, driven over pipes.

This is the default backend (Ray is optional here). It provides what the reference gets from
``RayWorkerGroup`` / ``RayResourcePool`` / ``create_colocated_worker_cls``
(verl/single_controller/ray/base.py:98-1098): rank environment for ``torch.distributed``
rendezvous, per-worker method execution with futures, colocated multi-role workers in one
process, per-role views (``spawn``), liveness checks, and detached re-attachment by name inside
one controller process.
"""

from __future__ import annotations

import atexit
import itertools
import multiprocessing as mp
import os
import pickle
import socket
import threading
import traceback
from concurrent.futures import Future
from typing import Any, Optional

from ..base.decorator import MAGIC_ATTR, Dispatch, Execute, register
from ..base.worker import Worker
from ..base.worker_group import ClassWithInitArgs, ResourcePool, WorkerGroup, func_generator

_CTX = mp.get_context("spawn")
_NAMED_GROUPS: dict[str, "MPWorkerGroup"] = {}


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class RemoteError(RuntimeError):
    """An exception raised inside a worker process, carried to the controller with its traceback."""


def _worker_main(conn, cls_blob: bytes, env: dict, name: str):
    os.environ.update({k: str(v) for k, v in env.items()})
    try:
        cia: ClassWithInitArgs = pickle.loads(cls_blob)
        worker = cia()
        conn.send(("ready", None, None))
    except BaseException as e:  # construction failed: report and exit
        conn.send(("init_error", None, "".join(traceback.format_exception(type(e), e, e.__traceback__))))
        return
    import asyncio
    import inspect

    loop = None
    while True:
        try:
            msg = conn.recv()
        except (EOFError, OSError):
            break
        kind, req_id, payload = msg
        if kind == "stop":
            break
        method, args, kwargs = payload
        try:
            fn = getattr(worker, method)
            out = fn(*args, **kwargs)
            if inspect.isawaitable(out):
                if loop is None:
                    loop = asyncio.new_event_loop()
                out = loop.run_until_complete(out)
            conn.send(("ok", req_id, out))
        except BaseException as e:
            tb = "".join(traceback.format_exception(type(e), e, e.__traceback__))
            try:
                conn.send(("err", req_id, (type(e).__name__, str(e), tb)))
            except Exception:
                break
            if isinstance(e, (KeyboardInterrupt, SystemExit)):
                break
    try:
        shutdown = getattr(worker, "shutdown", None)
        if callable(shutdown):
            shutdown()
    except Exception:
        pass


class _WorkerHandle:
    """Controller-side endpoint of one worker process."""

    def __init__(self, rank: int, name: str, cls_blob: bytes, env: dict):
        self.rank, self.name = rank, name
        self._parent, child = _CTX.Pipe()
        self.proc = _CTX.Process(target=_worker_main, args=(child, cls_blob, env, name), daemon=True, name=name)
        self.proc.start()
        child.close()
        self._pending: dict[int, Future] = {}
        self._ids = itertools.count()
        self._lock = threading.Lock()
        self._send_lock = threading.Lock()
        self._ready = Future()
        self._reader = threading.Thread(target=self._read_loop, daemon=True)
        self._reader.start()

    def _read_loop(self):
        while True:
            try:
                kind, req_id, payload = self._parent.recv()
            except (EOFError, OSError):
                err = RemoteError(f"worker {self.name} exited unexpectedly")
                if not self._ready.done():
                    self._ready.set_exception(err)
                with self._lock:
                    for f in self._pending.values():
                        if not f.done():
                            f.set_exception(err)
                    self._pending.clear()
                return
            if kind == "ready":
                self._ready.set_result(True)
            elif kind == "init_error":
                self._ready.set_exception(RemoteError(f"worker {self.name} failed to initialise:\n{payload}"))
            else:
                with self._lock:
                    fut = self._pending.pop(req_id, None)
                if fut is None:
                    continue
                if kind == "ok":
                    fut.set_result(payload)
                else:
                    etype, emsg, tb = payload
                    fut.set_exception(RemoteError(f"{etype} in worker {self.name}: {emsg}\n{tb}"))

    def wait_ready(self, timeout: Optional[float] = None):
        self._ready.result(timeout)

    def call(self, method: str, args, kwargs) -> Future:
        fut: Future = Future()
        req_id = next(self._ids)
        with self._lock:
            self._pending[req_id] = fut
        try:
            with self._send_lock:
                self._parent.send(("call", req_id, (method, args, kwargs)))
        except (OSError, ValueError) as e:
            with self._lock:
                self._pending.pop(req_id, None)
            fut.set_exception(RemoteError(f"worker {self.name} is gone: {e}"))
        return fut

    def is_alive(self) -> bool:
        return self.proc.is_alive()

    def stop(self, timeout: float = 5.0):
        try:
            with self._send_lock:
                self._parent.send(("stop", None, None))
        except Exception:
            pass
        self.proc.join(timeout)
        if self.proc.is_alive():
            self.proc.terminate()
            self.proc.join(2.0)

    def kill(self):
        self.proc.kill()

    def __repr__(self):
        return f"<worker {self.name} pid={self.proc.pid}>"


class MPResourcePool(ResourcePool):
    """Slots for worker processes. ``use_gpu`` pins rank i of a node to GPU i (CUDA_VISIBLE_DEVICES)."""

    def __init__(self, process_on_nodes=None, use_gpu: bool = True, name_prefix: str = "", max_colocate_count: int = 10,
                 detached: bool = False, accelerator_type: Optional[str] = None, gpu_offset: int = 0) -> None:
        super().__init__(process_on_nodes, max_colocate_count)
        self.use_gpu = use_gpu
        self.name_prefix = name_prefix or f"pool{next(_POOL_IDS)}"
        self.detached = detached
        self.accelerator_type = accelerator_type
        self.gpu_offset = gpu_offset
        self.pgs = None

    def get_placement_groups(self, *args, **kwargs):
        """Placement is implicit (local ranks); returns one pseudo group per node for API parity."""
        if self.pgs is None:
            self.pgs = [{"node": i, "bundles": n} for i, n in enumerate(self._store)]
        return self.pgs


_POOL_IDS = itertools.count()


def split_resource_pool(resource_pool: MPResourcePool, split_size) -> list[MPResourcePool]:
    """Split a single-node pool into sub-pools of the given sizes (int = equal parts)."""
    total = resource_pool.world_size
    sizes = [split_size] * (total // split_size) if isinstance(split_size, int) else list(split_size)
    assert sum(sizes) == total, f"split sizes {sizes} do not sum to {total}"
    out, off = [], resource_pool.gpu_offset
    for i, s in enumerate(sizes):
        out.append(MPResourcePool([s], use_gpu=resource_pool.use_gpu, name_prefix=f"{resource_pool.name_prefix}_s{i}",
                                  max_colocate_count=resource_pool.max_colocate_count, gpu_offset=off))
        off += s
    return out


def merge_resource_pool(rp1: MPResourcePool, rp2: MPResourcePool) -> MPResourcePool:
    assert rp1.use_gpu == rp2.use_gpu, "Both RayResourcePool must either use_gpu or not"
    assert rp1.max_colocate_count == rp2.max_colocate_count, "Both RayResourcePool must has the same max_colocate_count"
    return MPResourcePool(rp1.store + rp2.store, rp1.use_gpu, f"{rp1.name_prefix}_{rp2.name_prefix}",
                          rp1.max_colocate_count, gpu_offset=min(rp1.gpu_offset, rp2.gpu_offset))


class MPClassWithInitArgs(ClassWithInitArgs):
    def __init__(self, cls, *args, **kwargs) -> None:
        super().__init__(cls, *args, **kwargs)
        self._options: dict = {}
        self._additional_resource: dict = {}

    def set_additional_resource(self, additional_resource):
        self._additional_resource = additional_resource

    def update_options(self, options: dict):
        self._options.update(options)


class MPWorkerGroup(WorkerGroup):
    """Spawns ``resource_pool.world_size`` worker processes and binds the worker class's registered methods."""

    def __init__(self, resource_pool: MPResourcePool | None = None, ray_cls_with_init: MPClassWithInitArgs | None = None,
                 bin_pack: bool = True, name_prefix: str | None = None, detached: bool = False,
                 worker_names: list[str] | None = None, worker_handles: list | None = None, device_name: str = "cuda",
                 env: dict | None = None, **kwargs) -> None:
        super().__init__(resource_pool=resource_pool, **kwargs)
        self.ray_cls_with_init = ray_cls_with_init
        self.name_prefix = name_prefix or f"wg{next(_POOL_IDS)}"
        self.device_name = device_name
        self._extra_env = dict(env or {})
        self.sub_cls_name = ""
        self.profile_steps = kwargs.get("profile_steps")
        self.worker_nsight_options = kwargs.get("worker_nsight_options")
        if worker_handles is not None:  # a view on existing workers (spawn / from_detached)
            self._workers = list(worker_handles)
            self._worker_names = list(worker_names or [w.name for w in worker_handles])
            self._owns_workers = False
        else:
            assert resource_pool is not None and ray_cls_with_init is not None
            self._owns_workers = True
            self._init_with_resource_pool(resource_pool, ray_cls_with_init)
        if ray_cls_with_init is not None:
            self._bind_worker_method(ray_cls_with_init.cls, func_generator)
        self.wg_dict = None
        self.method_names: list[str] = []
        if detached:
            _NAMED_GROUPS[self.name_prefix] = self
        atexit.register(self.shutdown)

    # ------------------------------------------------------------------ lifecycle
    def _init_with_resource_pool(self, pool: MPResourcePool, cia: MPClassWithInitArgs):
        world = pool.world_size
        self._master_addr, self._master_port = "127.0.0.1", str(_free_port())
        blob = pickle.dumps(cia)
        local_sizes, local_ranks = pool.local_world_size_list(), pool.local_rank_list()
        use_gpu = getattr(pool, "use_gpu", False) and self.device_name == "cuda"
        for rank in range(world):
            env = {"WORLD_SIZE": world, "RANK": rank, "LOCAL_WORLD_SIZE": local_sizes[rank],
                   "LOCAL_RANK": local_ranks[rank], "MASTER_ADDR": self._master_addr, "MASTER_PORT": self._master_port,
                   "WG_PREFIX": self.name_prefix, "WG_BACKEND": "mp", "RAY_LOCAL_WORLD_SIZE": local_sizes[rank]}
            if use_gpu:
                env["CUDA_VISIBLE_DEVICES"] = str(getattr(pool, "gpu_offset", 0) + local_ranks[rank])
                env["LOCAL_RANK"] = 0  # each process sees exactly one device
            elif self.device_name == "cpu":
                env["CUDA_VISIBLE_DEVICES"] = ""
            env.update(self._extra_env)
            name = f"{self.name_prefix}{cia.cls.__name__}_{rank}"
            self._workers.append(_WorkerHandle(rank, name, blob, env))
            self._worker_names.append(name)
        for w in self._workers:
            w.wait_ready(timeout=float(os.environ.get("VERL_WORKER_START_TIMEOUT", 600)))

    def shutdown(self):
        if getattr(self, "_owns_workers", False):
            for w in self._workers:
                try:
                    w.stop()
                except Exception:
                    pass
            self._workers = []
            self._owns_workers = False

    def _is_worker_alive(self, worker) -> bool:
        return worker.is_alive()

    @property
    def worker_names(self):
        return self._worker_names

    @property
    def workers(self):
        return self._workers

    @property
    def master_address(self):
        return self._master_addr

    @property
    def master_port(self):
        return self._master_port

    @classmethod
    def from_detached(cls, name_prefix=None, worker_names=None, worker_handles=None, ray_cls_with_init=None, **kwargs):
        if worker_handles is None:
            src = _NAMED_GROUPS[name_prefix]
            worker_handles, worker_names = src._workers, src._worker_names
        return cls(resource_pool=None, ray_cls_with_init=ray_cls_with_init, name_prefix=name_prefix,
                   worker_names=worker_names, worker_handles=worker_handles, **kwargs)

    # ---------------------------------------------------------------- role views
    def spawn(self, prefix_set) -> dict[str, "MPWorkerGroup"]:
        """Per-role views of a colocated worker group: methods named ``{role}_{method}`` on the fused
        worker appear as ``method`` on the view returned for ``role``."""
        out = {}
        for prefix in prefix_set:
            view = self.from_detached(name_prefix=self.name_prefix, worker_names=self._worker_names,
                                      worker_handles=self._workers, ray_cls_with_init=self.ray_cls_with_init,
                                      device_name=self.device_name)
            pre = prefix + "_"
            for name in dir(view):
                if name.startswith(pre):
                    setattr(view, name[len(pre):], getattr(view, name))
            view.sub_cls_name = prefix
            out[prefix] = view
        return out

    def spawn_fused(self, prefix_set):
        return self.spawn(prefix_set)

    # ----------------------------------------------------------------- execution
    def _resolve(self, output):
        if isinstance(output, list):
            return [o.result() if isinstance(o, Future) else o for o in output]
        return output.result() if isinstance(output, Future) else output

    def _call_worker(self, worker, method_name, args, kwargs) -> Future:
        return worker.call(method_name, args, kwargs)

    def execute_rank_zero_async(self, method_name: str, *args, **kwargs):
        return self._call_worker(self._workers[0], method_name, args, kwargs)

    def execute_rank_zero_sync(self, method_name: str, *args, **kwargs):
        return self.execute_rank_zero_async(method_name, *args, **kwargs).result()

    def execute_rank_zero(self, method_name: str, *args, **kwargs):
        return self.execute_rank_zero_async(method_name, *args, **kwargs)

    def execute_all_async(self, method_name: str, *args, **kwargs) -> list[Future]:
        """If every argument is a list of length world_size, worker i gets element i; otherwise all
        workers get the same arguments."""
        n = len(self._workers)
        sliced = all(isinstance(a, list) for a in args) and all(isinstance(v, list) for v in kwargs.values()) and \
            all(len(a) == n for a in args) and all(len(v) == n for v in kwargs.values()) and (args or kwargs)
        futs = []
        for i, w in enumerate(self._workers):
            if sliced:
                a = tuple(x[i] for x in args)
                kw = {k: v[i] for k, v in kwargs.items()}
            else:
                a, kw = args, kwargs
            futs.append(self._call_worker(w, method_name, a, kw))
        return futs

    def execute_all_sync(self, method_name: str, *args, **kwargs):
        return [f.result() for f in self.execute_all_async(method_name, *args, **kwargs)]

    def execute_all(self, method_name: str, *args, **kwargs):
        return self.execute_all_async(method_name, *args, **kwargs)


# ------------------------------------------------------------------ colocated workers
def _bind_role_methods(cls, key: str, user_cls):
    """Expose every registered method of ``user_cls`` on the fused class as ``{key}_{method}``."""
    for name in dir(user_cls):
        try:
            method = getattr(user_cls, name)
            assert callable(method)
        except Exception:
            continue
        if not hasattr(method, MAGIC_ATTR):
            continue

        def make(name):
            import inspect

            if inspect.iscoroutinefunction(getattr(user_cls, name)):
                async def fn(self, *args, **kwargs):
                    return await getattr(self.worker_dict[key], name)(*args, **kwargs)
            else:
                def fn(self, *args, **kwargs):
                    return getattr(self.worker_dict[key], name)(*args, **kwargs)
            return fn

        fn = make(name)
        attrs = getattr(method, MAGIC_ATTR)
        setattr(fn, MAGIC_ATTR, attrs)
        try:
            setattr(cls, f"{key}_{name}", fn)
        except Exception as e:
            raise ValueError(f"Fail to set method_name {name}") from e


def create_colocated_worker_cls(class_dict: dict[str, ClassWithInitArgs]) -> MPClassWithInitArgs:
    """Fuse several role workers into one process: returns a ``WorkerDict`` class (wrapped with its
    init args) whose registered methods are the roles' methods prefixed by the role name."""
    return MPClassWithInitArgs(cls=_FusedFactory(dict(class_dict)))


class _FusedFactory:
    """Picklable stand-in for a dynamically created ``WorkerDict`` class: rebuilt inside the worker
    process from the (picklable) role classes. Acts as the ``cls`` of a ClassWithInitArgs."""

    def __init__(self, class_dict: dict[str, ClassWithInitArgs]):
        self.class_dict = class_dict
        self.__name__ = "WorkerDict"
        self._cls = None

    def _build(self):
        if self._cls is None:
            cls_dict = {k: v.cls for k, v in self.class_dict.items()}
            init_args = {k: (v.args, v.kwargs) for k, v in self.class_dict.items()}

            class WorkerDict(Worker):
                def __init__(inner):
                    super().__init__()
                    inner.worker_dict = {k: c(*init_args[k][0], **init_args[k][1]) for k, c in cls_dict.items()}

                def shutdown(inner):
                    for w in inner.worker_dict.values():
                        fn = getattr(w, "shutdown", None)
                        if callable(fn):
                            fn()

            for key, user_cls in cls_dict.items():
                _bind_role_methods(WorkerDict, key, user_cls)
            self._cls = WorkerDict
        return self._cls

    def __call__(self, *args, **kwargs):
        return self._build()(*args, **kwargs)

    def __getstate__(self):
        return {"class_dict": self.class_dict}

    def __setstate__(self, state):
        self.class_dict = state["class_dict"]
        self.__name__ = "WorkerDict"
        self._cls = None

    # dir()/getattr() on the factory expose the fused class's methods for controller-side binding
    def __dir__(self):
        return dir(self._build())

    def __getattr__(self, name):
        if name.startswith("__") or name in ("class_dict", "_cls"):
            raise AttributeError(name)
        return getattr(self._build(), name)

    @property
    def __mro__(self):
        return self._build().__mro__


class ResourcePoolManager:
    """Maps roles to named resource pools (verl/single_controller/ray/base.py:167-221)."""

    def __init__(self, resource_pool_spec: dict[str, list[int]], mapping: dict, use_gpu: bool = True):
        self.resource_pool_spec = resource_pool_spec
        self.mapping = mapping
        self.use_gpu = use_gpu
        self.resource_pool_dict: dict[str, MPResourcePool] = {}

    def create_resource_pool(self):
        off = 0
        for name, process_on_nodes in self.resource_pool_spec.items():
            self.resource_pool_dict[name] = MPResourcePool(process_on_nodes=process_on_nodes, use_gpu=self.use_gpu,
                                                           max_colocate_count=3, name_prefix=name, gpu_offset=off)
            off += sum(process_on_nodes) if self.use_gpu else 0
        self._check_resource_available()

    def get_resource_pool(self, role) -> MPResourcePool:
        return self.resource_pool_dict[self.mapping[role]]

    def get_n_gpus(self) -> int:
        return sum(n for spec in self.resource_pool_spec.values() for n in spec)

    def _check_resource_available(self):
        if not self.use_gpu:
            return
        try:
            import torch

            avail = torch.cuda.device_count()
        except Exception:
            avail = 0
        need = self.get_n_gpus()
        if avail and need > avail:
            raise ValueError(f"Total available GPUs {avail} is less than total desired GPUs {need}")
