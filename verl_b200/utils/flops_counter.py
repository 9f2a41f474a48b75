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


def _get(c, name, default=None):
    v = getattr(c, name, None) if not isinstance(c, dict) else c.get(name)
    return default if v is None else v


def _text(c):
    """The language-model part of a (possibly multimodal) config."""
    t = _get(c, "text_config")
    return t if t is not None else c


class FlopsCounter:
    """``estimate_flops(batch_seqlens, delta_time, images_seqlens=None) -> (achieved TFLOP/s, device peak TFLOP/s)``.

    Architectures (by ``model_type``): dense decoders (llama, qwen2, qwen3, mistral, seed_oss, ...), Qwen MoE, DeepSeek-V3
    (multi-head latent attention, shared + routed experts, leading dense layers), Gemma-3 and GPT-OSS (sliding-window
    layers cost ``s * min(s, window)`` instead of ``s^2``), Apertus (two-matrix MLP), and the Qwen VL families (text
    decoder + vision tower over ``images_seqlens`` patches). An unknown type counts as 0, as in the reference
    (verl/utils/flops_counter.py:534)."""

    def __init__(self, config):
        self.config = config
        mt = _get(config, "model_type", "qwen2")
        dense = ("qwen2", "llama", "qwen3", "mistral", "mimo", "seed_oss", "minicpmv", "minicpmo", "glm4", "internlm2",
                 "deepseek", "gemma", "gemma2", "phi3", "olmo2")
        table = {m: self._dense for m in dense}
        table.update({"qwen3_moe": self._moe, "qwen2_moe": self._moe, "deepseek_v3": self._deepseek_v3,
                      "gemma3": self._sliding, "gemma3_text": self._sliding, "gpt_oss": self._gpt_oss,
                      "apertus": self._apertus, "qwen2_vl": self._vl, "qwen2_5_vl": self._vl, "qwen3_vl": self._vl,
                      "qwen3_vl_moe": self._vl, "kimi_vl": self._deepseek_v3})
        self._fn = table.get(mt, self._unknown)

    # ---- building blocks ----
    @staticmethod
    def _hd(c):
        return _get(c, "head_dim") or c.hidden_size // c.num_attention_heads

    def _attn_params(self, c) -> float:
        hd = self._hd(c)
        q, kv = c.num_attention_heads * hd, _get(c, "num_key_value_heads", c.num_attention_heads) * hd
        return c.hidden_size * (q + 2 * kv + q)

    def _attn_flops(self, c, batch_seqlens, layers=None, window=None) -> float:
        """Score + value FLOPs, forward and backward (12 per head-dim element and key-query pair, no causal
        discount); a sliding window caps the keys per query."""
        if window:
            sq = sum(s * min(s, window) for s in batch_seqlens)
        else:
            sq = sum(s * s for s in batch_seqlens)
        return 12 * sq * self._hd(c) * c.num_attention_heads * (c.num_hidden_layers if layers is None else layers)

    # ---- families ----
    def _dense(self, tokens_sum, batch_seqlens, **kw) -> float:
        c = _text(self.config)
        mlp = c.hidden_size * c.intermediate_size * 3
        emb = c.vocab_size * c.hidden_size * 2
        dense = (mlp + self._attn_params(c)) * c.num_hidden_layers + emb
        return 6 * dense * tokens_sum + self._attn_flops(c, batch_seqlens)

    def _apertus(self, tokens_sum, batch_seqlens, **kw) -> float:
        c = _text(self.config)
        mlp = c.hidden_size * c.intermediate_size * 2  # up and down only: the activation is not gated
        emb = c.vocab_size * c.hidden_size * 2
        dense = (mlp + self._attn_params(c)) * c.num_hidden_layers + emb
        return 6 * dense * tokens_sum + self._attn_flops(c, batch_seqlens)

    def _moe_mlp(self, c) -> float:
        E = _get(c, "num_experts", None) or _get(c, "num_local_experts", 0)
        k = _get(c, "num_experts_per_tok", None) or _get(c, "experts_per_token", 1)
        inter = _get(c, "moe_intermediate_size", None) or c.intermediate_size
        shared = _get(c, "shared_expert_intermediate_size", 0) or 0
        return c.hidden_size * inter * k * 3 + c.hidden_size * E + c.hidden_size * shared * 3

    def _moe(self, tokens_sum, batch_seqlens, **kw) -> float:
        c = _text(self.config)
        emb = c.vocab_size * c.hidden_size * 2
        dense = (self._moe_mlp(c) + self._attn_params(c)) * c.num_hidden_layers + emb
        return 6 * dense * tokens_sum + self._attn_flops(c, batch_seqlens)

    def _layer_windows(self, c):
        """Per layer: the sliding window (None = full attention)."""
        L, w = c.num_hidden_layers, _get(c, "sliding_window")
        types = _get(c, "layer_types")
        if types:
            return [w if "sliding" in str(t) else None for t in types]
        pat = _get(c, "sliding_window_pattern")
        if w and pat:
            return [None if (i + 1) % pat == 0 else w for i in range(L)]
        return [None] * L

    def _windowed_attn(self, c, batch_seqlens) -> float:
        wins = self._layer_windows(c)
        n_full = sum(1 for w in wins if not w)
        total = self._attn_flops(c, batch_seqlens, layers=n_full)
        for w in {w for w in wins if w}:
            total += self._attn_flops(c, batch_seqlens, layers=sum(1 for x in wins if x == w), window=w)
        return total

    def _sliding(self, tokens_sum, batch_seqlens, **kw) -> float:
        c = _text(self.config)
        mlp = c.hidden_size * c.intermediate_size * 3
        emb = c.vocab_size * c.hidden_size * 2
        dense = (mlp + self._attn_params(c)) * c.num_hidden_layers + emb
        return 6 * dense * tokens_sum + self._windowed_attn(c, batch_seqlens)

    def _gpt_oss(self, tokens_sum, batch_seqlens, **kw) -> float:
        c = _text(self.config)
        emb = c.vocab_size * c.hidden_size * 2
        dense = (self._moe_mlp(c) + self._attn_params(c)) * c.num_hidden_layers + emb
        return 6 * dense * tokens_sum + self._windowed_attn(c, batch_seqlens)

    def _deepseek_v3(self, tokens_sum, batch_seqlens, **kw) -> float:
        c = _text(self.config)
        H, nh = c.hidden_size, c.num_attention_heads
        nope, rope, vd = _get(c, "qk_nope_head_dim", 128), _get(c, "qk_rope_head_dim", 64), _get(c, "v_head_dim", 128)
        qk = nope + rope
        q_lora, kv_lora = _get(c, "q_lora_rank"), _get(c, "kv_lora_rank", 512)
        attn = (H * q_lora + q_lora * nh * qk) if q_lora else H * nh * qk
        attn += H * (kv_lora + rope) + kv_lora * nh * (nope + vd) + nh * vd * H
        first_dense = _get(c, "first_k_dense_replace", 0)
        freq = _get(c, "moe_layer_freq", 1) or 1
        L = c.num_hidden_layers
        moe_layers = sum(1 for i in range(L) if i >= first_dense and i % freq == 0)
        k = _get(c, "num_experts_per_tok", 8)
        moe_mlp = H * c.moe_intermediate_size * 3 * (k + (_get(c, "n_shared_experts", 0) or 0)) + H * _get(c, "n_routed_experts", 0)
        dense_mlp = H * c.intermediate_size * 3
        emb = c.vocab_size * H * 2
        dense = attn * L + moe_mlp * moe_layers + dense_mlp * (L - moe_layers) + emb
        sq = sum(s * s for s in batch_seqlens)
        return 6 * dense * tokens_sum + 6 * sq * (qk + vd) * nh * L

    def _vit_flops(self, images_seqlens) -> float:
        """Vision tower of the Qwen VL families over ``images_seqlens`` patches per image (before the 2 x 2 merge)."""
        v = _get(self.config, "vision_config")
        if v is None:  # this repo's ModelConfig keeps the vision tower's description among its extra fields
            v = (_get(self.config, "extra") or {}).get("vision_config")
        if not v or not images_seqlens:
            return 0.0
        d = _get(v, "embed_dim", None) or _get(v, "hidden_size")
        depth = _get(v, "depth", None) or _get(v, "num_hidden_layers")
        inter = _get(v, "intermediate_size")
        mlp = 3 * d * inter if inter and _get(self.config, "model_type") == "qwen2_5_vl" else 2 * d * (inter or int(d * _get(v, "mlp_ratio", 4)))
        merge = _get(v, "spatial_merge_size", 2) ** 2
        out = _get(v, "out_hidden_size", None) or _get(_text(self.config), "hidden_size")  # width of the language model
        patch = _get(v, "in_channels", _get(v, "in_chans", 3)) * _get(v, "temporal_patch_size", 2) * _get(v, "patch_size", 14) ** 2
        mergers = 1 + len(_get(v, "deepstack_visual_indexes", None) or ())  # Qwen3-VL: one more merger per deepstack tap
        per_patch = (4 * d * d + mlp) * depth + patch * d + mergers * (d * merge * d * merge + d * merge * out) / merge
        tokens = sum(images_seqlens)
        heads_dim = d  # heads x head_dim
        return 6 * per_patch * tokens + 12 * sum(s * s for s in images_seqlens) * heads_dim * depth

    def _vl(self, tokens_sum, batch_seqlens, images_seqlens=None, **kw) -> float:
        t = _text(self.config)
        text = self._moe(tokens_sum, batch_seqlens) if _get(t, "num_experts") else self._dense(tokens_sum, batch_seqlens)
        return text + self._vit_flops(images_seqlens)

    @staticmethod
    def _unknown(tokens_sum, batch_seqlens, **kw) -> float:
        return 0.0

    def estimate_flops(self, batch_seqlens, delta_time: float, images_seqlens=None):
        if isinstance(batch_seqlens, (int, float)):
            batch_seqlens = [int(batch_seqlens)]
        tokens = sum(batch_seqlens)
        achieved = self._fn(tokens, batch_seqlens, images_seqlens=images_seqlens) / max(delta_time, 1e-9) / 1e12
        return achieved, get_device_flops()
