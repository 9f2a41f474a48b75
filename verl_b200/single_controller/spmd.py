"""In-process worker group for SPMD launches (``torchrun``: one controller replica per rank).

Every rank runs the same trainer loop on its own shard of the batch; a "remote" call is a local method
call on the rank's worker, so batches never leave the GPU's process and no driver gathers them. This is
the launch mode of ``bench.py`` and of ``python -m torch.distributed.run -m verl_b200.trainer.main_ppo``.
The reference has no such mode (its SFT trainer is SPMD, its RL trainers are Ray-driven).
"""

from __future__ import annotations

from .base.decorator import MAGIC_ATTR
from .base.worker_group import ClassWithInitArgs, ResourcePool, WorkerGroup


class SPMDResourcePool(ResourcePool):
    def __init__(self, process_on_nodes=None, use_gpu: bool = True, name_prefix: str = "", max_colocate_count: int = 10,
                 **kwargs):
        super().__init__(process_on_nodes or [1], max_colocate_count)
        self.use_gpu, self.name_prefix = use_gpu, name_prefix


class SPMDWorkerGroup(WorkerGroup):
    is_spmd = True

    def __init__(self, resource_pool=None, ray_cls_with_init: ClassWithInitArgs | None = None, worker=None,
                 prefix: str = "", **kwargs):
        super().__init__(resource_pool=None)
        self.worker = worker if worker is not None else ray_cls_with_init()
        self._workers = [self.worker]
        self._prefix = prefix
        self._bind(prefix)

    def _bind(self, prefix: str):
        pre = prefix + "_" if prefix else ""
        for name in dir(type(self.worker)):
            try:
                method = getattr(type(self.worker), name)
            except Exception:
                continue
            if not callable(method) or not hasattr(method, MAGIC_ATTR):
                continue
            if pre and not name.startswith(pre):
                continue
            attrs = getattr(method, MAGIC_ATTR)
            bound = getattr(self.worker, name)
            if not attrs.get("blocking", True):
                bound = _as_future(bound)
            setattr(self, name[len(pre):], bound)

    @property
    def world_size(self) -> int:
        return 1

    def spawn(self, prefix_set):
        return {p: SPMDWorkerGroup(worker=self.worker, prefix=p) for p in prefix_set}

    def execute_all_sync(self, method_name, *args, **kwargs):
        return [getattr(self.worker, method_name)(*args, **kwargs)]

    execute_all = execute_all_sync

    def shutdown(self):
        fn = getattr(self.worker, "shutdown", None)
        if callable(fn):
            fn()


class _Done:
    def __init__(self, value):
        self._v = value

    def result(self, timeout=None):
        return self._v

    def get(self):
        return self._v


def _as_future(fn):
    def call(*args, **kwargs):
        return _Done(fn(*args, **kwargs))

    return call


def create_colocated_worker_cls_spmd(class_dict: dict[str, ClassWithInitArgs]) -> ClassWithInitArgs:
    from .mp.worker_group import _FusedFactory

    return ClassWithInitArgs(cls=_FusedFactory(dict(class_dict)))
