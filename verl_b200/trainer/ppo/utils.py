"""Roles and config-derived switches (verl/trainer/ppo/utils.py:1-97)."""

from __future__ import annotations

import warnings
from enum import Enum


class Role(Enum):
    Actor = 0
    Rollout = 1
    ActorRollout = 2
    Critic = 3
    RefPolicy = 4
    RewardModel = 5
    ActorRolloutRef = 6
    Env = 7

    def __str__(self):
        return self._get_role_string()

    def _get_role_string(self):
        return {Role.Actor: "actor", Role.Rollout: "rollout", Role.ActorRollout: "actor_rollout", Role.Critic: "critic",
                Role.RefPolicy: "ref", Role.RewardModel: "rm", Role.ActorRolloutRef: "actor_rollout_ref",
                Role.Env: "env"}[self]

    @classmethod
    def from_string(cls, name: str):
        table = {"actor": cls.Actor, "rollout": cls.Rollout, "actor_rollout": cls.ActorRollout, "critic": cls.Critic,
                 "ref": cls.RefPolicy, "rm": cls.RewardModel, "actor_rollout_ref": cls.ActorRolloutRef, "env": cls.Env}
        if name.lower() not in table:
            raise ValueError(f"No Role found for string: {name}")
        return table[name.lower()]


def need_reference_policy(config) -> bool:
    """A reference policy is needed when KL enters the reward or the loss."""
    return bool(config.algorithm.get("use_kl_in_reward", False) or config.actor_rollout_ref.actor.get("use_kl_loss", False))


def need_reward_model(config) -> bool:
    return bool(config.reward_model.get("enable", False))


def need_critic(config) -> bool:
    """``critic.enable`` decides when set; otherwise a critic is needed for GAE only."""
    enable = config.critic.get("enable", None)
    if enable is not None:
        return bool(enable)
    if config.algorithm.adv_estimator == "gae":
        return True
    warnings.warn("Disabled critic as algorithm.adv_estimator != gae. If it is not intended, please set critic.enable=True",
                  stacklevel=2)
    return False
