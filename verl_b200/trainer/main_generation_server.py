"""Offline generation through standalone rollout servers (role of verl/trainer/main_generation_server.py:40-170).

Starts ``rollout.num_replicas`` standalone replicas (one native engine + HTTP server each), spreads the prompts over
them round-robin, sends every sample as its own request to ``/v1/completions`` (token-in / token-out; the servers
batch them continuously) and writes ``responses`` next to each input row.

    python -m verl_b200.trainer.main_generation_server model.path=preset:tiny-qwen2 data.path=prompts.jsonl \\
        data.output_path=out.jsonl rollout.n=4 rollout.response_length=128
"""

from __future__ import annotations

import asyncio
import copy
import json
import os
import sys

import numpy as np
import torch

from ..utils.config import compose_from_dict
from .main_generation import DEFAULTS as _BASE

DEFAULTS = copy.deepcopy(_BASE)
DEFAULTS["rollout"].update(num_replicas=1, server_address="127.0.0.1", max_concurrency=256, request_timeout=600)


def _engine_factory(config, dev):
    from ..models.transformer import CausalLM
    from ..rollout import NativeRolloutEngine
    from ..workers.engine_workers import resolve_model_config

    model_cfg, state = resolve_model_config(config.model)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    rc = config.rollout

    def build():
        model = CausalLM(model_cfg, dtype=dtype, device=dev)
        if state is not None:
            model.load_state_dict({k: v.to(dtype) for k, v in state.items()}, strict=False)
        else:
            model.init_weights(int(rc.seed))
        return NativeRolloutEngine(model, max_num_seqs=int(rc.max_num_seqs),
                                   max_model_len=int(rc.prompt_length) + int(rc.response_length),
                                   max_num_batched_tokens=int(rc.max_num_batched_tokens),
                                   gpu_memory_utilization=float(rc.gpu_memory_utilization),
                                   enforce_eager=bool(rc.enforce_eager) or dev.type != "cuda", seed=int(rc.seed))

    return model_cfg, build


async def start_server(config):
    """Returns (replicas, ["host:port", ...], serving tasks)."""
    from ..workers.rollout.replica import get_rollout_replica_class
    from ..workers.rollout.utils import run_unvicorn

    rc = config.rollout
    n_rep = int(rc.num_replicas)
    cls = get_rollout_replica_class("native")
    replicas, addresses, tasks = [], [], []
    for r in range(n_rep):
        if config.trainer.device == "cuda" and torch.cuda.is_available():
            dev = torch.device("cuda", r % torch.cuda.device_count())
        else:
            dev = torch.device("cpu")
        _, factory = _engine_factory(config, dev)
        rep = cls(replica_rank=r, config=rc, model_config=config.model, engine_factory=factory)
        await rep.init_standalone()
        port, task = await run_unvicorn(rep.server_handle.build_app(), None, str(rc.server_address))
        replicas.append(rep)
        addresses.append(f"{rc.server_address}:{port}")
        tasks.append(task)
    return replicas, addresses, tasks


async def submit_request(session, address: str, prompt_ids: list[int], sampling: dict, timeout: float) -> list[int]:
    import aiohttp

    async with session.post(f"http://{address}/v1/completions", json={"prompt": prompt_ids, **sampling},
                            timeout=aiohttp.ClientTimeout(total=timeout)) as resp:
        resp.raise_for_status()
        body = await resp.json()
    return body["choices"][0]["token_ids"]


async def generate(config, addresses: list[str], prompts: list[list[int]], n: int) -> list[list[list[int]]]:
    import aiohttp

    rc = config.rollout
    sampling = {"temperature": float(rc.temperature) if rc.do_sample else 0.0, "top_p": float(rc.top_p),
                "max_tokens": int(rc.response_length)}
    sem = asyncio.Semaphore(int(rc.max_concurrency))

    async with aiohttp.ClientSession() as session:
        async def one(i, ids):
            async with sem:
                return await submit_request(session, addresses[i % len(addresses)], ids, sampling, float(rc.request_timeout))

        flat = await asyncio.gather(*[one(i, ids) for i, ids in enumerate(prompts) for _ in range(n)])
    return [flat[i * n:(i + 1) * n] for i in range(len(prompts))]


async def run_generation_server(config) -> list[dict]:
    from ..utils.dataset.rl_dataset import _read_rows
    from ..workers.engine_workers import resolve_model_config
    from .main_ppo import build_tokenizer

    model_cfg, _ = resolve_model_config(config.model)
    tok = build_tokenizer(config.model, model_cfg)
    rows = _read_rows(config.data.path)
    if config.data.max_samples and int(config.data.max_samples) > 0:
        rows = rows[: int(config.data.max_samples)]
    rc = config.rollout
    prompts = []
    for r in rows:
        p = r[config.data.prompt_key]
        chat = p if isinstance(p, (list, np.ndarray)) else [{"role": "user", "content": str(p)}]
        prompts.append([int(t) for t in tok.apply_chat_template(list(chat), add_generation_prompt=True, tokenize=True)][-int(rc.prompt_length):])
    replicas, addresses, tasks = await start_server(config)
    try:
        outs = await generate(config, addresses, prompts, int(config.data.n_samples or rc.n))
    finally:
        for t in tasks:
            t.server.should_exit = True
        await asyncio.gather(*tasks, return_exceptions=True)
        for rep in replicas:
            rep.server_handle.shutdown()
    result = []
    for r, samples in zip(rows, outs):
        keep = {k: v for k, v in r.items() if isinstance(v, (str, int, float, list, dict))}
        result.append({**keep, "responses": [tok.decode(s, skip_special_tokens=True) for s in samples]})
    path = os.path.expanduser(str(config.data.output_path))
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    if path.endswith(".parquet"):
        import pandas as pd

        pd.DataFrame(result).to_parquet(path)
    else:
        with open(path, "w") as f:
            for r in result:
                f.write(json.dumps(r) + "\n")
    return result


def main(argv=None):
    cfg = compose_from_dict(DEFAULTS, list(sys.argv[1:] if argv is None else argv))
    return asyncio.run(run_generation_server(cfg))


if __name__ == "__main__":
    main()
