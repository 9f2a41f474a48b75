from .base import BasePPORewardModel

__all__ = ["BasePPORewardModel"]
