"""Controller-side handle on a group of workers.

Counterpart of verl/single_controller/base/worker_group.py:27-255. ``WorkerGroup`` binds every
``@register``-ed method of the worker class as a controller-side method whose call is
dispatch -> execute on the workers -> collect. Backends (multiprocess, SPMD/in-process, Ray when
present) implement ``execute_all`` / ``execute_rank_zero`` (+ ``_async`` variants).
"""

from __future__ import annotations

import logging
import os
import signal
import threading
import time
from typing import Any, Callable

from ...protocol import _PAD_KEY, DataProto, DataProtoFuture, unpad_dataproto
from .decorator import MAGIC_ATTR, Dispatch, get_predefined_dispatch_fn, get_predefined_execute_fn

logger = logging.getLogger(__name__)


class ResourcePool:
    """``process_on_nodes[i]`` worker slots on node i; ``max_colocate_count`` worker groups may share a slot."""

    def __init__(self, process_on_nodes=None, max_colocate_count: int = 10, n_gpus_per_node: int = 8) -> None:
        self._store = list(process_on_nodes or [])
        self.max_colocate_count = max_colocate_count
        self.n_gpus_per_node = n_gpus_per_node

    def add_node(self, process_count):
        self._store.append(process_count)

    @property
    def world_size(self):
        return sum(self._store)

    def __call__(self) -> Any:
        return self._store

    @property
    def store(self):
        return self._store

    def local_world_size_list(self) -> list[int]:
        return [n for n in self._store for _ in range(n)]

    def local_rank_list(self) -> list[int]:
        return [i for n in self._store for i in range(n)]


class ClassWithInitArgs:
    """A worker class together with the arguments of its (deferred, remote) construction."""

    def __init__(self, cls, *args, **kwargs) -> None:
        self.cls = cls
        self.args = args
        self.kwargs = kwargs
        self.fused_worker_used = False

    def __call__(self) -> Any:
        return self.cls(*self.args, **self.kwargs)


def check_workers_alive(workers: list, is_alive: Callable, gap_time: float = 1) -> None:
    """Liveness loop run in a daemon thread: a dead worker aborts the controller (SIGABRT)."""
    while True:
        for w in workers:
            if not is_alive(w):
                logger.warning(f"worker {w} is not alive, sending signal to main thread")
                signal.raise_signal(signal.SIGABRT)
        time.sleep(gap_time)


class WorkerGroup:
    fused_worker_execute_fn_name = "_fuw_execute"

    def __init__(self, resource_pool: ResourcePool | None, **kwargs) -> None:
        self._is_init_with_detached_workers = resource_pool is None
        self.fused_worker_used = False
        self._procecss_dispatch_config = resource_pool() if resource_pool is not None else None
        self._workers: list = []
        self._worker_names: list = []
        self._dispatch_info: dict = {}
        self._collect_info: dict = {}
        self._master_addr = None
        self._master_port = None
        self._checker_thread: threading.Thread | None = None

    def _is_worker_alive(self, worker) -> bool:
        raise NotImplementedError("WorkerGroup._is_worker_alive called, should be implemented in derived class.")

    def _block_until_all_workers_alive(self) -> None:
        while not all(self._is_worker_alive(w) for w in self._workers):
            time.sleep(0.1)

    def start_worker_aliveness_check(self, every_n_seconds: float = 1) -> None:
        self._block_until_all_workers_alive()
        self._checker_thread = threading.Thread(target=check_workers_alive,
                                                args=(self._workers, self._is_worker_alive, every_n_seconds), daemon=True)
        self._checker_thread.start()

    @property
    def world_size(self) -> int:
        return len(self._workers)

    def _query_dispatch_info(self, mesh_name: str):
        return self.execute_all_sync("_query_dispatch_info", mesh_name)

    def _query_collect_info(self, mesh_name: str):
        return self.execute_all_sync("_query_collect_info", mesh_name)

    # ------------------------------------------------------------------ binding
    def _bind_worker_method(self, user_defined_cls, func_generator) -> list[str]:
        """Create a controller-side method for every worker method that carries ``@register`` metadata."""
        bound = []
        for name in dir(user_defined_cls):
            try:
                method = getattr(user_defined_cls, name)
                assert callable(method)
            except Exception:
                continue
            if not hasattr(method, MAGIC_ATTR):
                continue
            attrs = getattr(method, MAGIC_ATTR)
            assert isinstance(attrs, dict), f"attribute of {name} should be a dictionary. Got {type(attrs)}"
            mode = attrs["dispatch_mode"]
            if isinstance(mode, Dispatch):
                fns = get_predefined_dispatch_fn(mode)
                dispatch_fn, collect_fn = fns["dispatch_fn"], fns["collect_fn"]
            else:
                dispatch_fn, collect_fn = mode["dispatch_fn"], mode["collect_fn"]
            exec_name = get_predefined_execute_fn(attrs["execute_mode"])["execute_fn_name"]
            try:
                execute_fn = getattr(self, exec_name)
                assert callable(execute_fn)
            except Exception:
                print(f"execute_fn {exec_name} is invalid")
                raise
            func = func_generator(self, name, dispatch_fn=dispatch_fn, collect_fn=collect_fn, execute_fn=execute_fn,
                                  blocking=attrs["blocking"])
            try:
                setattr(self, name, func)
                bound.append(name)
            except Exception as e:
                raise ValueError(f"Fail to set method_name {name}") from e
        return bound


def func_generator(self, method_name, dispatch_fn, collect_fn, execute_fn, blocking):
    """dispatch -> execute -> (resolve) -> collect -> strip auto-padding."""

    class Functor:
        def __call__(this, *args, **kwargs):
            args, kwargs = dispatch_fn(self, *args, **kwargs)
            pad = kwargs.pop(_PAD_KEY, None)
            output = execute_fn(method_name, *args, **kwargs)
            if blocking:
                output = self._resolve(output)
            output = collect_fn(self, output)
            if pad and isinstance(output, DataProto):
                output = unpad_dataproto(output, pad_size=pad)
            return output

    return type(method_name, (Functor,), {})()
