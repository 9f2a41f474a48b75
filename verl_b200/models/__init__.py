from .config import PRESETS, ModelConfig, preset
from .transformer import CausalLM, PackedBatch, build_model

__all__ = ["ModelConfig", "PRESETS", "preset", "CausalLM", "PackedBatch", "build_model"]
