"""Native ops of the framework. CUDA tensors run on the hand-written sm_100a kernels in
``verl_b200/csrc`` (loaded through :mod:`verl_b200.ops._lib`); CPU tensors take plain-torch
reference paths that exist for the CPU test tier."""

from . import _lib
from .attention import attention_varlen, decode_workspace, kv_cache_write, paged_decode_attention
from .gemm import gemm, linear
from .lmhead import lmhead_logprob_entropy
from .nn import embedding, rmsnorm, rope_qkv, rope_tables, swiglu
from .rl import (PPO_METRIC_NAMES, adamw_step, clip_coef, decode_advance, gae, grpo_advantage, ppo_loss_fused, sample,
                 sumsq_into)

__all__ = [
    "_lib", "gemm", "linear", "lmhead_logprob_entropy", "embedding", "rmsnorm", "rope_qkv", "rope_tables", "swiglu",
    "attention_varlen", "paged_decode_attention", "kv_cache_write", "decode_workspace", "ppo_loss_fused", "gae",
    "grpo_advantage", "sample", "decode_advance", "adamw_step", "sumsq_into", "clip_coef", "PPO_METRIC_NAMES",
]
