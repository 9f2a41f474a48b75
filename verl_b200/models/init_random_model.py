"""Write a randomly initialised model of a given architecture as an HF checkpoint (config.json + safetensors), e.g.
for synthetic benchmarks without network access; role of the reference's ``scripts/init_random_model.py``.

    python -m verl_b200.models.init_random_model --preset qwen2.5-0.5b --out /tmp/rand-qwen [--seed 0] \\
        [--override num_hidden_layers=4 hidden_size=512]
"""

from __future__ import annotations

import argparse

import torch

from .config import preset
from .hf_io import save_hf_checkpoint
from .transformer import build_model


def _value(text: str):
    for cast in (int, float):
        try:
            return cast(text)
        except ValueError:
            pass
    return {"true": True, "false": False, "none": None}.get(text.lower(), text)


def main(argv=None) -> str:
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "float16"])
    ap.add_argument("--override", nargs="*", default=[], help="ModelConfig fields, key=value")
    a = ap.parse_args(argv)
    cfg = preset(a.preset, **{k: _value(v) for k, v in (kv.split("=", 1) for kv in a.override)})
    model = build_model(cfg, dtype=torch.float32, seed=a.seed)
    save_hf_checkpoint(cfg, dict(model.state_dict()), a.out, dtype=getattr(torch, a.dtype))
    n = sum(p.numel() for p in model.parameters())
    print(f"wrote {n / 1e6:.1f}M parameters ({cfg.model_type}, {cfg.num_hidden_layers} layers) to {a.out}")
    return a.out


if __name__ == "__main__":
    main()
