"""Names of the reference's Ray backend (verl/single_controller/ray/base.py).

Ray is not a dependency of this framework: the multiprocess backend implements the same
contract, and these names resolve to it so code written against ``verl.single_controller.ray``
runs unchanged on one box (one NVSwitch domain is the whole machine; there is no Ray actor back end).
"""

from ..mp.worker_group import MPClassWithInitArgs as RayClassWithInitArgs
from ..mp.worker_group import MPResourcePool as RayResourcePool
from ..mp.worker_group import MPWorkerGroup as RayWorkerGroup
from ..mp.worker_group import ResourcePoolManager, create_colocated_worker_cls, merge_resource_pool, split_resource_pool

__all__ = ["RayResourcePool", "RayWorkerGroup", "RayClassWithInitArgs", "create_colocated_worker_cls",
           "ResourcePoolManager", "split_resource_pool", "merge_resource_pool"]
