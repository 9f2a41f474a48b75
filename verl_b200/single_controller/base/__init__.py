from .decorator import Dispatch, Execute, make_nd_compute_dataproto_dispatch_fn, register
from .worker import Worker
from .worker_group import ClassWithInitArgs, ResourcePool, WorkerGroup

__all__ = ["Worker", "WorkerGroup", "ClassWithInitArgs", "ResourcePool", "register", "Dispatch", "Execute",
           "make_nd_compute_dataproto_dispatch_fn"]
