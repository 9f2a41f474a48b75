"""Architecture description shared by the training engine, the rollout engine and the
checkpoint code. Mirrors the HF ``config.json`` fields of the supported families
(Llama, Qwen2/2.5, Qwen3, Qwen3-MoE); the reference gets these models from
``transformers`` (verl/utils/model.py:103-127)."""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any

_ARCH_TO_TYPE = {
    "LlamaForCausalLM": "llama",
    "MistralForCausalLM": "llama",
    "Qwen2ForCausalLM": "qwen2",
    "Qwen3ForCausalLM": "qwen3",
    "Qwen3MoeForCausalLM": "qwen3_moe",
    "ApertusForCausalLM": "apertus",
    "Qwen2VLForConditionalGeneration": "qwen2_vl",
    "Qwen2_5_VLForConditionalGeneration": "qwen2_5_vl",
    "Qwen3VLForConditionalGeneration": "qwen3_vl",
    "Qwen3VLMoeForConditionalGeneration": "qwen3_vl_moe",
    "LlamaForTokenClassification": "llama",
    "Qwen2ForTokenClassification": "qwen2",
    "Qwen3ForTokenClassification": "qwen3",
}
_TYPE_TO_ARCH = {"llama": "LlamaForCausalLM", "qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM",
                 "qwen3_moe": "Qwen3MoeForCausalLM", "qwen2_vl": "Qwen2VLForConditionalGeneration",
                 "qwen2_5_vl": "Qwen2_5_VLForConditionalGeneration", "apertus": "ApertusForCausalLM",
                 "qwen3_vl": "Qwen3VLForConditionalGeneration", "qwen3_vl_moe": "Qwen3VLMoeForConditionalGeneration"}
_VL_TYPES = ("qwen2_vl", "qwen2_5_vl", "qwen3_vl", "qwen3_vl_moe")


@dataclass
class ModelConfig:
    model_type: str = "qwen2"
    vocab_size: int = 152064
    hidden_size: int = 3584
    intermediate_size: int = 18944
    num_hidden_layers: int = 28
    num_attention_heads: int = 28
    num_key_value_heads: int = 4
    head_dim: int | None = None
    rope_theta: float = 1e6
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = False
    attention_bias: bool | None = None  # None -> family default (qwen2: True)
    qk_norm: bool | None = None  # None -> family default (qwen3*, apertus: True)
    # "silu": gated SwiGLU MLP (gate / up / down); "xielu": Apertus' two-matrix MLP with the learnable xIELU activation
    hidden_act: str | None = None
    # MoE (qwen3_moe)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    router_aux_loss_coef: float = 0.0
    # token-classification / value head
    num_labels: int = 0
    bos_token_id: int | None = None
    eos_token_id: int | None = 2
    pad_token_id: int | None = None
    extra: dict = field(default_factory=dict)

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.attention_bias is None:
            self.attention_bias = self.model_type in ("qwen2", "qwen2_vl", "qwen2_5_vl")
        if self.qk_norm is None:
            self.qk_norm = self.model_type in ("qwen3", "qwen3_moe", "apertus", "qwen3_vl", "qwen3_vl_moe")
        if self.hidden_act is None:
            self.hidden_act = "xielu" if self.model_type == "apertus" else "silu"

    # ------------------------------------------------------------------ derived
    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def mlp_gated(self) -> bool:
        return self.hidden_act != "xielu"

    # vision-language models (Qwen2-VL family): the decoder fields above describe the language model; the vision tower,
    # the placeholder token ids and the multimodal RoPE sections live in ``extra``
    @property
    def is_vl(self) -> bool:
        return bool(self.extra.get("vision_config"))

    @property
    def mrope_section(self):
        return self.extra.get("mrope_section")

    @property
    def mrope_interleaved(self) -> bool:
        """Qwen3-VL: the frequencies of the three axes alternate (T H W T H W ... T T) instead of lying in three
        consecutive sections."""
        return bool(self.extra.get("mrope_interleaved", False))

    @property
    def image_token_id(self) -> int:
        return int(self.extra.get("image_token_id", 151655))

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def num_parameters(self, include_embedding: bool = True) -> int:
        H, L = self.hidden_size, self.num_hidden_layers
        attn = H * (self.q_size + 2 * self.kv_size) + self.q_size * H
        if self.attention_bias:
            attn += self.q_size + 2 * self.kv_size
        if self.qk_norm:
            attn += 2 * self.head_dim
        if self.is_moe:
            mlp = self.num_experts * 3 * H * self.moe_intermediate_size + H * self.num_experts
        else:
            mlp = (3 if self.mlp_gated else 2) * H * self.intermediate_size + (0 if self.mlp_gated else 2)
        total = L * (attn + mlp + 2 * H) + H
        if include_embedding:
            total += self.vocab_size * H * (1 if self.tie_word_embeddings else 2)
        return total

    # --------------------------------------------------------------- (de)serialise
    @classmethod
    def from_hf_dict(cls, d: dict[str, Any]) -> "ModelConfig":
        mt = d.get("model_type")
        if mt is None:
            archs = d.get("architectures") or ["Qwen2ForCausalLM"]
            mt = _ARCH_TO_TYPE.get(archs[0], "qwen2")
        if mt in _VL_TYPES:  # language-model fields are nested under text_config in recent HF versions
            top = {k: v for k, v in d.items() if k not in ("text_config", "vision_config")}
            flat = dict(top)
            flat.update(d.get("text_config") or {})
            rope = flat.get("rope_scaling") or flat.get("rope_parameters") or {}
            flat["model_type"] = mt
            extra_vl = {"vision_config": dict(d.get("vision_config") or {}),
                        "mrope_section": list(rope.get("mrope_section") or []) or None}
            if rope.get("mrope_interleaved") or mt in ("qwen3_vl", "qwen3_vl_moe"):
                extra_vl["mrope_interleaved"] = True
            if "rope_theta" not in flat and rope.get("rope_theta"):
                flat["rope_theta"] = rope["rope_theta"]
            for k in ("image_token_id", "video_token_id", "vision_start_token_id", "vision_end_token_id"):
                if k in top:
                    extra_vl[k] = top[k]
            d = {k: v for k, v in flat.items() if k not in ("rope_scaling", "rope_parameters", "image_token_id",
                                                            "video_token_id", "vision_start_token_id", "vision_end_token_id")}
            d["_vl_extra"] = extra_vl
        else:
            # text models: recent HF versions nest theta and the scaling rule under rope_parameters
            rope = d.get("rope_parameters") or d.get("rope_scaling") or None
            if isinstance(rope, dict):
                d = dict(d)
                if d.get("rope_theta") is None and rope.get("rope_theta") is not None:
                    d["rope_theta"] = rope["rope_theta"]
                kind = rope.get("rope_type") or rope.get("type") or "default"
                d.pop("rope_parameters", None)
                d.pop("rope_scaling", None)
                if kind != "default":
                    d["rope_scaling"] = {k: v for k, v in rope.items() if k != "rope_theta"}
        known = {f for f in cls.__dataclass_fields__}
        may_be_none = ("eos_token_id", "pad_token_id", "bos_token_id", "head_dim", "attention_bias", "qk_norm", "hidden_act")
        kw = {k: v for k, v in d.items() if k in known and k != "extra" and (v is not None or k in may_be_none)}
        kw["model_type"] = mt
        if "num_local_experts" in d and "num_experts" not in d:
            kw["num_experts"] = d["num_local_experts"]
        eos = kw.get("eos_token_id")
        if isinstance(eos, list):
            kw["eos_token_id"] = eos[0]
        cfg = cls(**kw)
        if cfg.is_moe and (d.get("mlp_only_layers") or int(d.get("decoder_sparse_step") or 1) != 1):
            raise NotImplementedError("mixture-of-experts stacks with dense layers in between (mlp_only_layers, "
                                      "decoder_sparse_step != 1) are not supported: every layer is sparse here")
        cfg.extra = {k: v for k, v in d.items() if k not in known and k != "_vl_extra"}
        cfg.extra.update(d.get("_vl_extra") or {})
        return cfg

    @classmethod
    def from_pretrained(cls, path: str | Path) -> "ModelConfig":
        p = Path(path)
        if p.is_dir():
            p = p / "config.json"
        return cls.from_hf_dict(json.loads(p.read_text()))

    def to_hf_dict(self) -> dict[str, Any]:
        d = asdict(self)
        extra = d.pop("extra")
        if self.model_type in _VL_TYPES:
            moe_keys = () if self.is_moe else ("num_experts", "num_experts_per_tok", "moe_intermediate_size", "norm_topk_prob",
                                               "router_aux_loss_coef")
            text = {k: v for k, v in d.items() if k not in moe_keys + ("num_labels",)}
            text["model_type"] = self.model_type + "_text"
            text["rope_scaling"] = {"type": "mrope", "mrope_section": list(extra.get("mrope_section") or [])}
            if self.model_type in ("qwen3_vl", "qwen3_vl_moe"):
                text["rope_scaling"] = {"rope_type": "default", "mrope_section": list(extra.get("mrope_section") or []),
                                        "mrope_interleaved": True, "rope_theta": self.rope_theta}
            out = {"architectures": [_TYPE_TO_ARCH[self.model_type]], "model_type": self.model_type, "torch_dtype": "bfloat16",
                   "text_config": text, "vision_config": dict(extra.get("vision_config") or {}),
                   "tie_word_embeddings": self.tie_word_embeddings}
            for k in ("image_token_id", "video_token_id", "vision_start_token_id", "vision_end_token_id"):
                if k in extra:
                    out[k] = extra[k]
            return out
        arch = _TYPE_TO_ARCH.get(self.model_type, "Qwen2ForCausalLM")
        if self.num_labels:
            arch = arch.replace("ForCausalLM", "ForTokenClassification")
        d["architectures"] = [arch]
        d["torch_dtype"] = "bfloat16"
        if not self.is_moe:
            for k in ("num_experts", "num_experts_per_tok", "moe_intermediate_size", "norm_topk_prob",
                      "router_aux_loss_coef"):
                d.pop(k)
        if not self.num_labels:
            d.pop("num_labels")
        d.update({k: v for k, v in extra.items() if k not in d})
        return d

    def save_pretrained(self, path: str | Path) -> None:
        p = Path(path)
        p.mkdir(parents=True, exist_ok=True)
        (p / "config.json").write_text(json.dumps(self.to_hf_dict(), indent=2))


# Named architectures used by the benchmarks and tests (random-init, no download needed).
PRESETS: dict[str, dict] = {
    "tiny-qwen2": dict(model_type="qwen2", vocab_size=2048, hidden_size=256, intermediate_size=688,
                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, rope_theta=1e6,
                       tie_word_embeddings=True, eos_token_id=2),
    "qwen2.5-0.5b": dict(model_type="qwen2", vocab_size=151936, hidden_size=896, intermediate_size=4864,
                         num_hidden_layers=24, num_attention_heads=14, num_key_value_heads=2, rope_theta=1e6,
                         tie_word_embeddings=True, eos_token_id=151645),
    "qwen2.5-7b": dict(model_type="qwen2", vocab_size=152064, hidden_size=3584, intermediate_size=18944,
                       num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4, rope_theta=1e6,
                       eos_token_id=151645),
    "qwen2.5-32b": dict(model_type="qwen2", vocab_size=152064, hidden_size=5120, intermediate_size=27648,
                        num_hidden_layers=64, num_attention_heads=40, num_key_value_heads=8, rope_theta=1e6,
                        eos_token_id=151645),
    "qwen3-30b-a3b": dict(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048, intermediate_size=6144,
                          num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4, head_dim=128,
                          rope_theta=1e6, num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768,
                          eos_token_id=151645),
    "tiny-qwen3-moe": dict(model_type="qwen3_moe", vocab_size=2048, hidden_size=256, intermediate_size=512,
                           num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                           num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128, eos_token_id=2),
    "tiny-qwen2-vl": dict(model_type="qwen2_vl", vocab_size=2048, hidden_size=256, intermediate_size=512,
                          num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, rope_theta=1e6, eos_token_id=2,
                          extra={"vision_config": dict(depth=2, embed_dim=64, hidden_size=256, num_heads=2, mlp_ratio=2,
                                                       in_channels=3, patch_size=4, spatial_merge_size=2,
                                                       temporal_patch_size=2),
                                 "mrope_section": [8, 12, 12], "image_token_id": 2000, "video_token_id": 2001,
                                 "vision_start_token_id": 2002}),
    "tiny-qwen2.5-vl": dict(model_type="qwen2_5_vl", vocab_size=2048, hidden_size=256, intermediate_size=512,
                            num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, rope_theta=1e6, eos_token_id=2,
                            extra={"vision_config": dict(depth=3, hidden_size=64, out_hidden_size=256, intermediate_size=96,
                                                         num_heads=2, in_channels=3, patch_size=4, spatial_merge_size=2,
                                                         temporal_patch_size=2, window_size=16, fullatt_block_indexes=[1],
                                                         hidden_act="silu"),
                                   "mrope_section": [8, 12, 12], "image_token_id": 2000, "video_token_id": 2001,
                                   "vision_start_token_id": 2002}),
    "tiny-qwen3-vl": dict(model_type="qwen3_vl", vocab_size=2048, hidden_size=256, intermediate_size=512,
                          num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=64, rope_theta=5e6,
                          eos_token_id=2,
                          extra={"vision_config": dict(depth=4, hidden_size=64, out_hidden_size=256, intermediate_size=96,
                                                       num_heads=2, in_channels=3, patch_size=4, spatial_merge_size=2,
                                                       temporal_patch_size=2, num_position_embeddings=64,
                                                       deepstack_visual_indexes=[0, 2], hidden_act="gelu_pytorch_tanh"),
                                 "mrope_section": [12, 10, 10], "mrope_interleaved": True, "image_token_id": 2000,
                                 "video_token_id": 2001, "vision_start_token_id": 2002}),
    "tiny-qwen3-vl-moe": dict(model_type="qwen3_vl_moe", vocab_size=2048, hidden_size=256, intermediate_size=512,
                              num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=64, rope_theta=5e6,
                              num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128, eos_token_id=2,
                              extra={"vision_config": dict(depth=3, hidden_size=64, out_hidden_size=256, intermediate_size=96,
                                                           num_heads=2, in_channels=3, patch_size=4, spatial_merge_size=2,
                                                           temporal_patch_size=2, num_position_embeddings=64,
                                                           deepstack_visual_indexes=[0, 1], hidden_act="gelu_pytorch_tanh"),
                                     "mrope_section": [12, 10, 10], "mrope_interleaved": True, "image_token_id": 2000,
                                     "video_token_id": 2001, "vision_start_token_id": 2002}),
    "qwen3-vl-30b-a3b": dict(model_type="qwen3_vl_moe", vocab_size=151936, hidden_size=2048, intermediate_size=6144,
                             num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4, head_dim=128, rope_theta=5e6,
                             num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768, eos_token_id=151645,
                             max_position_embeddings=262144,
                             extra={"vision_config": dict(depth=27, hidden_size=1152, out_hidden_size=2048,
                                                          intermediate_size=4304, num_heads=16, in_channels=3, patch_size=16,
                                                          spatial_merge_size=2, temporal_patch_size=2,
                                                          num_position_embeddings=2304, deepstack_visual_indexes=[8, 16, 24],
                                                          hidden_act="gelu_pytorch_tanh"),
                                    "mrope_section": [24, 20, 20], "mrope_interleaved": True, "image_token_id": 151655,
                                    "video_token_id": 151656, "vision_start_token_id": 151652}),
    "qwen3-vl-8b": dict(model_type="qwen3_vl", vocab_size=151936, hidden_size=4096, intermediate_size=12288,
                        num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128, rope_theta=5e6,
                        eos_token_id=151645, max_position_embeddings=262144,
                        extra={"vision_config": dict(depth=27, hidden_size=1152, out_hidden_size=4096, intermediate_size=4304,
                                                     num_heads=16, in_channels=3, patch_size=16, spatial_merge_size=2,
                                                     temporal_patch_size=2, num_position_embeddings=2304,
                                                     deepstack_visual_indexes=[8, 16, 24], hidden_act="gelu_pytorch_tanh"),
                               "mrope_section": [24, 20, 20], "mrope_interleaved": True, "image_token_id": 151655,
                               "video_token_id": 151656, "vision_start_token_id": 151652}),
    "qwen2.5-vl-7b": dict(model_type="qwen2_5_vl", vocab_size=152064, hidden_size=3584, intermediate_size=18944,
                          num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4, rope_theta=1e6,
                          eos_token_id=151645,
                          extra={"vision_config": dict(depth=32, hidden_size=1280, out_hidden_size=3584, intermediate_size=3420,
                                                       num_heads=16, in_channels=3, patch_size=14, spatial_merge_size=2,
                                                       temporal_patch_size=2, window_size=112,
                                                       fullatt_block_indexes=[7, 15, 23, 31], hidden_act="silu"),
                                 "mrope_section": [16, 24, 24], "image_token_id": 151655, "video_token_id": 151656,
                                 "vision_start_token_id": 151652}),
    "qwen2-vl-7b": dict(model_type="qwen2_vl", vocab_size=152064, hidden_size=3584, intermediate_size=18944,
                        num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4, rope_theta=1e6,
                        eos_token_id=151645,
                        extra={"vision_config": dict(depth=32, embed_dim=1280, hidden_size=3584, num_heads=16, mlp_ratio=4,
                                                     in_channels=3, patch_size=14, spatial_merge_size=2,
                                                     temporal_patch_size=2),
                               "mrope_section": [16, 24, 24], "image_token_id": 151655, "video_token_id": 151656,
                               "vision_start_token_id": 151652}),
    "tiny-apertus": dict(model_type="apertus", vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, rope_theta=1e6, rms_norm_eps=1e-5, eos_token_id=2),
    "apertus-8b": dict(model_type="apertus", vocab_size=131072, hidden_size=4096, intermediate_size=21504,
                       num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, rope_theta=1.2e7,
                       rms_norm_eps=1e-5, eos_token_id=2, max_position_embeddings=65536,
                       extra={"rope_scaling": {"rope_type": "llama3", "factor": 8.0, "original_max_position_embeddings": 8192,
                                               "low_freq_factor": 1.0, "high_freq_factor": 4.0}}),
    "llama-3-8b": dict(model_type="llama", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                       num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, rope_theta=5e5,
                       rms_norm_eps=1e-5, eos_token_id=128001),
}


def preset(name: str, **overrides) -> ModelConfig:
    kw = dict(PRESETS[name])
    kw.update(overrides)
    return ModelConfig(**kw)
