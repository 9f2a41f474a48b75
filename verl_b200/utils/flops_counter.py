"""Analytical FLOPs per step and MFU (verl/utils/flops_counter.py: ``_DEVICE_FLOPS`` :22-40,
``_estimate_qwen2_flops`` :88, ``FlopsCounter.estimate_flops`` :582).

Forward+backward of a decoder-only transformer costs 6 FLOPs per (dense parameter, token) plus
12 * layers * q_size * sum(seqlen^2) for attention (forward 2x2, backward 2x, no causal discount — the same
convention as the reference, so MFU numbers compare).
"""

from __future__ import annotations

import torch

_DEVICE_FLOPS = {
    "CPU": 448e9, "GB200": 2.5e15, "B200": 2.25e15, "MI300X": 1336e12, "H100": 989e12, "H800": 989e12, "H200": 989e12,
    "A100": 312e12, "A800": 312e12, "L40S": 362.05e12, "L40": 181.05e12, "A40": 149.7e12, "L20": 119.5e12,
    "H20": 148e12, "910B": 354e12, "Ascend910": 354e12, "RTX 3070 Ti": 21.75e12,
}


def get_device_flops(unit: str = "T", device_name: str | None = None) -> float:
    if device_name is None:
        device_name = torch.cuda.get_device_name() if torch.cuda.is_available() else "CPU"
    flops = float("inf")
    for key in ("GB200", "B200", "MI300X", "H100", "H800", "H200", "A100", "A800", "L40S", "L40", "A40", "L20", "H20",
                "910B", "Ascend910", "RTX 3070 Ti", "CPU"):
        if key in device_name:
            flops = _DEVICE_FLOPS[key]
            break
    return flops / {"B": 1e9, "K": 1e3, "M": 1e6, "G": 1e9, "T": 1e12, "P": 1e15}[unit]


class FlopsCounter:
    """``estimate_flops(batch_seqlens, delta_time) -> (achieved TFLOP/s, device peak TFLOP/s)``."""

    def __init__(self, config):
        self.config = config
        mt = getattr(config, "model_type", "qwen2")
        self._fn = {"qwen3_moe": self._moe, "qwen2_moe": self._moe}.get(mt, self._dense)

    def _attn_flops(self, c, batch_seqlens) -> float:
        sq = sum(s * s for s in batch_seqlens)
        hd = getattr(c, "head_dim", None) or c.hidden_size // c.num_attention_heads
        return 12 * sq * hd * c.num_attention_heads * c.num_hidden_layers

    def _dense(self, tokens_sum, batch_seqlens) -> float:
        c = self.config
        hd = getattr(c, "head_dim", None) or c.hidden_size // c.num_attention_heads
        q, kv = c.num_attention_heads * hd, c.num_key_value_heads * hd
        mlp = c.hidden_size * c.intermediate_size * 3
        attn = c.hidden_size * (q + 2 * kv + q)
        emb = c.vocab_size * c.hidden_size * 2
        dense = (mlp + attn) * c.num_hidden_layers + emb
        return 6 * dense * tokens_sum + self._attn_flops(c, batch_seqlens)

    def _moe(self, tokens_sum, batch_seqlens) -> float:
        c = self.config
        hd = getattr(c, "head_dim", None) or c.hidden_size // c.num_attention_heads
        q, kv = c.num_attention_heads * hd, c.num_key_value_heads * hd
        mlp = c.hidden_size * c.moe_intermediate_size * c.num_experts_per_tok * 3 + c.hidden_size * c.num_experts
        attn = c.hidden_size * (q + 2 * kv + q)
        emb = c.vocab_size * c.hidden_size * 2
        dense = (mlp + attn) * c.num_hidden_layers + emb
        return 6 * dense * tokens_sum + self._attn_flops(c, batch_seqlens)

    def estimate_flops(self, batch_seqlens, delta_time: float):
        if isinstance(batch_seqlens, (int, float)):
            batch_seqlens = [int(batch_seqlens)]
        tokens = sum(batch_seqlens)
        achieved = self._fn(tokens, batch_seqlens) / max(delta_time, 1e-9) / 1e12
        return achieved, get_device_flops()
