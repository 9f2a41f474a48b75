"""Offline batch generation: prompts file -> n sampled responses per prompt -> parquet / jsonl.

    python -m verl_b200.trainer.main_generation model.path=preset:tiny-qwen2 data.path=prompts.jsonl \\
        data.output_path=out.jsonl rollout.n=4 rollout.response_length=128

Role of verl/trainer/main_generation.py:1-154 (and ``main_generation_server.py``, which does the same through the
server endpoints: here the engine is in process, the async server is ``verl_b200.workers.rollout.async_server``).
"""

from __future__ import annotations

import json
import os
import sys

import numpy as np
import torch

from ..utils.config import ConfigDict, compose_from_dict


DEFAULTS = {
    "model": {"path": "preset:tiny-qwen2", "tokenizer_path": None, "trust_remote_code": False},
    "data": {"path": None, "prompt_key": "prompt", "n_samples": None, "output_path": "generation.jsonl", "batch_size": 128,
             "max_samples": -1},
    "rollout": {"n": 1, "temperature": 1.0, "top_k": -1, "top_p": 1.0, "prompt_length": 1024, "response_length": 512,
                "do_sample": True, "gpu_memory_utilization": 0.6, "max_num_seqs": 256, "max_num_batched_tokens": 8192,
                "enforce_eager": False, "seed": 0},
    "trainer": {"device": "cuda"},
}


def run_generation(config) -> list[dict]:
    from ..rollout import NativeRolloutEngine, SamplingParams
    from ..models.transformer import CausalLM
    from ..utils.dataset.rl_dataset import _read_rows
    from ..workers.engine_workers import resolve_model_config
    from .main_ppo import build_tokenizer

    dev = torch.device("cuda" if config.trainer.device == "cuda" and torch.cuda.is_available() else "cpu")
    model_cfg, state = resolve_model_config(config.model)
    tok = build_tokenizer(config.model, model_cfg)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    model = CausalLM(model_cfg, dtype=dtype, device=dev)
    if state is not None:
        model.load_state_dict({k: v.to(dtype) for k, v in state.items()}, strict=False)
    else:
        model.init_weights(int(config.rollout.seed))
    rc = config.rollout
    eng = NativeRolloutEngine(model, max_num_seqs=int(rc.max_num_seqs), max_model_len=int(rc.prompt_length) + int(rc.response_length),
                              max_num_batched_tokens=int(rc.max_num_batched_tokens),
                              gpu_memory_utilization=float(rc.gpu_memory_utilization),
                              enforce_eager=bool(rc.enforce_eager) or dev.type != "cuda", seed=int(rc.seed))
    rows = _read_rows(config.data.path)
    if config.data.max_samples and int(config.data.max_samples) > 0:
        rows = rows[: int(config.data.max_samples)]
    n = int(config.data.n_samples or rc.n)
    sp = SamplingParams(temperature=float(rc.temperature) if rc.do_sample else 0.0, top_k=int(rc.top_k), top_p=float(rc.top_p),
                        max_tokens=int(rc.response_length))
    out = []
    bs = int(config.data.batch_size)
    for lo in range(0, len(rows), bs):
        chunk = rows[lo : lo + bs]
        prompts = []
        for r in chunk:
            p = r[config.data.prompt_key]
            chat = p if isinstance(p, (list, np.ndarray)) else [{"role": "user", "content": str(p)}]
            ids = list(tok.apply_chat_template(list(chat), add_generation_prompt=True, tokenize=True))[-int(rc.prompt_length):]
            prompts.extend([ids] * n)
        res = eng.generate(prompts, sp)
        for i, r in enumerate(chunk):
            texts = [tok.decode(o.token_ids, skip_special_tokens=True) for o in res[i * n : (i + 1) * n]]
            out.append({**{k: v for k, v in r.items() if isinstance(v, (str, int, float, list, dict))}, "responses": texts})
    path = os.path.expanduser(str(config.data.output_path))
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    if path.endswith(".parquet"):
        import pandas as pd

        pd.DataFrame(out).to_parquet(path)
    else:
        with open(path, "w") as f:
            for r in out:
                f.write(json.dumps(r) + "\n")
    return out


def main(argv=None):
    cfg = compose_from_dict(DEFAULTS, list(sys.argv[1:] if argv is None else argv))
    run_generation(cfg)


if __name__ == "__main__":
    main()
