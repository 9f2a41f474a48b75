from .base import ClassWithInitArgs, ResourcePool, Worker, WorkerGroup

__all__ = ["Worker", "WorkerGroup", "ClassWithInitArgs", "ResourcePool"]
