"""Architecture registry (verl/models/registry.py:43-63): HF ``architectures`` name -> the native model family.

The reference maps an architecture to Megatron ``Parallel*ForCausalLMRmPadPP`` classes; here every supported family is
one :class:`CausalLM` parameterised by :class:`ModelConfig`, so the registry resolves to a builder instead."""

from __future__ import annotations

from functools import partial
from typing import Callable, Optional

_ARCH_TO_FAMILY = {
    "LlamaForCausalLM": "llama",
    "MistralForCausalLM": "llama",
    "Qwen2ForCausalLM": "qwen2",
    "Qwen3ForCausalLM": "qwen3",
    "Qwen3MoeForCausalLM": "qwen3_moe",
    "LlamaForTokenClassification": "llama",
    "Qwen2ForTokenClassification": "qwen2",
    "Qwen3ForTokenClassification": "qwen3",
}


class ModelRegistry:
    @staticmethod
    def load_model_cls(model_arch: str, value: bool = False) -> Optional[Callable]:
        """Returns ``build(cfg, dtype=..., device=...)`` for the architecture (with a value head if ``value``)."""
        if model_arch not in _ARCH_TO_FAMILY:
            return None
        from .transformer import build_model

        return partial(build_model, value_head=value)

    @staticmethod
    def family(model_arch: str) -> Optional[str]:
        return _ARCH_TO_FAMILY.get(model_arch)

    @staticmethod
    def get_supported_archs() -> list[str]:
        return list(_ARCH_TO_FAMILY)
