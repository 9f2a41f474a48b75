from .base import BasePPOActor
from .dp_actor import DataParallelPPOActor

__all__ = ["BasePPOActor", "DataParallelPPOActor"]
