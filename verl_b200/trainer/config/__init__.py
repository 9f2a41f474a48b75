"""Typed algorithm / trainer configs (verl/trainer/config/algorithm.py, config.py)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from ...base_config import BaseConfig

__all__ = ["KLControlConfig", "PFPPOConfig", "FilterGroupsConfig", "RolloutCorrectionConfig", "AlgoConfig",
           "CheckpointConfig", "ProfileConfig", "BaseModelConfig"]


@dataclass
class KLControlConfig(BaseConfig):
    type: str = "fixed"
    kl_coef: float = 0.001
    horizon: int = 10000
    target_kl: float = 0.1


@dataclass
class PFPPOConfig(BaseConfig):
    reweight_method: str = "pow"
    weight_pow: float = 2.0


@dataclass
class FilterGroupsConfig(BaseConfig):
    """DAPO dynamic sampling: keep only prompt groups whose ``metric`` is not identical across samples;
    keep generating until a full train batch is collected or ``max_num_gen_batches`` is reached."""

    enable: bool = False
    metric: Optional[str] = None
    max_num_gen_batches: int = 0


@dataclass
class RolloutCorrectionConfig(BaseConfig):
    """Importance-sampling / rejection-sampling correction between rollout and training policies."""

    rollout_is: Optional[str] = None
    rollout_is_threshold: float = 2.0
    rollout_rs: Optional[str] = None
    rollout_rs_threshold: Optional[Any] = None
    bypass_mode: bool = False
    loss_type: str = "ppo_clip"
    rollout_is_batch_normalize: bool = False

    # ---- presets (same names as the reference) ----
    @classmethod
    def decoupled_token_is(cls, threshold: float = 2.0):
        return cls(rollout_is="token", rollout_is_threshold=threshold)

    @classmethod
    def decoupled_seq_is(cls, threshold: float = 2.0):
        return cls(rollout_is="sequence", rollout_is_threshold=threshold)

    @classmethod
    def decoupled_seq_is_rs(cls, is_threshold: float = 2.0, rs_threshold="0.5_2.0"):
        return cls(rollout_is="sequence", rollout_is_threshold=is_threshold, rollout_rs="seq_sum_k1",
                   rollout_rs_threshold=rs_threshold)

    @classmethod
    def decoupled_geo_rs(cls, rs_threshold="0.999_1.001"):
        return cls(rollout_rs="seq_mean_k1", rollout_rs_threshold=rs_threshold)

    @classmethod
    def decoupled_k3_rs(cls, rs_threshold: float = 0.01):
        return cls(rollout_rs="seq_mean_k3", rollout_rs_threshold=rs_threshold)

    @classmethod
    def decoupled_k3_rs_token_tis(cls, is_threshold: float = 2.0, rs_threshold: float = 0.01):
        return cls(rollout_is="token", rollout_is_threshold=is_threshold, rollout_rs="seq_mean_k3",
                   rollout_rs_threshold=rs_threshold)

    @classmethod
    def bypass_ppo_clip(cls):
        return cls(bypass_mode=True, loss_type="ppo_clip")

    @classmethod
    def bypass_ppo_clip_geo_rs(cls, rs_threshold="0.999_1.001"):
        return cls(bypass_mode=True, loss_type="ppo_clip", rollout_rs="seq_mean_k1", rollout_rs_threshold=rs_threshold)

    @classmethod
    def bypass_ppo_clip_k3_rs(cls, rs_threshold: float = 0.01):
        return cls(bypass_mode=True, loss_type="ppo_clip", rollout_rs="seq_mean_k3", rollout_rs_threshold=rs_threshold)

    @classmethod
    def bypass_pg_is(cls, threshold: float = 2.0):
        return cls(bypass_mode=True, loss_type="reinforce", rollout_is="sequence", rollout_is_threshold=threshold)

    @classmethod
    def bypass_pg_geo_rs(cls, rs_threshold="0.999_1.001"):
        return cls(bypass_mode=True, loss_type="reinforce", rollout_rs="seq_mean_k1", rollout_rs_threshold=rs_threshold)

    @classmethod
    def bypass_pg_geo_rs_seq_tis(cls, is_threshold: float = 2.0, rs_threshold="0.999_1.001"):
        return cls(bypass_mode=True, loss_type="reinforce", rollout_is="sequence", rollout_is_threshold=is_threshold,
                   rollout_rs="seq_mean_k1", rollout_rs_threshold=rs_threshold)

    @classmethod
    def bypass_pg_geo_rs_token_tis(cls, is_threshold: float = 2.0, rs_threshold="0.999_1.001"):
        return cls(bypass_mode=True, loss_type="reinforce", rollout_is="token", rollout_is_threshold=is_threshold,
                   rollout_rs="seq_mean_k1", rollout_rs_threshold=rs_threshold)

    @classmethod
    def disabled(cls):
        return cls()


@dataclass
class AlgoConfig(BaseConfig):
    gamma: float = 1.0
    lam: float = 1.0
    adv_estimator: str = "gae"
    norm_adv_by_std_in_grpo: bool = True
    use_kl_in_reward: bool = False
    kl_penalty: str = "kl"
    kl_ctrl: KLControlConfig = field(default_factory=KLControlConfig)
    use_pf_ppo: bool = False
    pf_ppo: Any = field(default_factory=dict)
    filter_groups: Optional[Any] = None
    rollout_correction: Optional[Any] = None


@dataclass
class CheckpointConfig(BaseConfig):
    save_contents: list = field(default_factory=lambda: ["model", "optimizer", "extra"])
    load_contents: list = field(default_factory=lambda: ["model", "optimizer", "extra"])
    async_save: bool = False


@dataclass
class ProfileConfig(BaseConfig):
    profile_ranks: Optional[list] = None
    step_start: int = -1
    step_end: int = -1
    save_path: Optional[str] = None


@dataclass
class BaseModelConfig(BaseConfig):
    path: str = "~/models/deepseek-llm-7b-chat"
    tokenizer_path: Optional[str] = None
    override_config: dict = field(default_factory=dict)
    external_lib: Optional[str] = None
    trust_remote_code: bool = False
