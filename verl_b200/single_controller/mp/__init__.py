from .worker_group import (MPClassWithInitArgs, MPResourcePool, MPWorkerGroup, RemoteError, ResourcePoolManager,
                           create_colocated_worker_cls, merge_resource_pool, split_resource_pool)

__all__ = ["MPWorkerGroup", "MPResourcePool", "MPClassWithInitArgs", "create_colocated_worker_cls",
           "ResourcePoolManager", "split_resource_pool", "merge_resource_pool", "RemoteError"]
