"""Reward loop: token bucket, rate-limited manager, batch manager (role of the reference's
tests/experimental/reward_loop/test_async_token_bucket_on_cpu.py and test_rate_limited_reward_manager_on_cpu.py)."""

import asyncio
import time

import numpy as np
import torch

from verl_b200.experimental.reward_loop import AsyncTokenBucket, RateLimitedRewardManager, RewardLoopManager
from verl_b200.protocol import DataProto
from verl_b200.utils.config import to_config
from verl_b200.utils.tokenizer import IntTokenizer


def test_token_bucket_rate():
    async def go():
        b = AsyncTokenBucket(rate_limit=50.0, max_tokens=5.0)
        t0 = time.perf_counter()
        for _ in range(15):  # 5 for free, 10 more at 50/s = 0.2 s
            await b.acquire(1.0)
        return time.perf_counter() - t0

    dt = asyncio.run(go())
    assert 0.15 < dt < 0.6


def test_token_bucket_oversized_request():
    async def go():
        b = AsyncTokenBucket(rate_limit=100.0, max_tokens=10.0)
        t0 = time.perf_counter()
        await b.acquire(30.0)  # 10 there, 20 more at 100/s
        return time.perf_counter() - t0, b.tokens

    dt, tokens = asyncio.run(go())
    assert 0.15 < dt < 0.5 and tokens < 0


def _batch(n=6, P=4, R=5):
    ids = torch.randint(3, 50, (n, P + R))
    mask = torch.ones(n, P + R, dtype=torch.long)
    mask[0, -2:] = 0
    nt = {"data_source": np.array(["synthetic/even_fraction"] * n, dtype=object),
          "reward_model": np.array([{"ground_truth": None}] * n, dtype=object)}
    return DataProto.from_dict(tensors={"prompts": ids[:, :P], "responses": ids[:, P:], "input_ids": ids, "attention_mask": mask},
                               non_tensors=nt)


def test_rate_limited_manager_concurrency():
    RateLimitedRewardManager.reset_class()
    active, peak = [0], [0]

    async def slow_score(data_source, solution_str, ground_truth, extra_info=None):
        active[0] += 1
        peak[0] = max(peak[0], active[0])
        await asyncio.sleep(0.02)
        active[0] -= 1
        return 1.0

    cfg = to_config({"reward_model": {"max_concurrent": 2, "max_rpm": None, "max_tpm": None, "timeout": 5.0}})
    data = _batch(6)

    async def go():
        m = RateLimitedRewardManager(cfg, IntTokenizer(64), compute_score=slow_score)
        return await asyncio.gather(*[m.run_single(data[i : i + 1]) for i in range(len(data))])

    out = asyncio.run(go())
    assert peak[0] <= 2 and all(o["reward_score"] == 1.0 for o in out)
    RateLimitedRewardManager.reset_class()


def test_reward_loop_manager_scores_last_token():
    cfg = to_config({"reward_model": {"reward_manager": "naive", "num_workers": 2, "enable": False},
                     "custom_reward_function": {"path": None}})
    mgr = RewardLoopManager(cfg, IntTokenizer(64))
    try:
        data = _batch(5)
        out = mgr.compute_rm_score(data)
        rm = out.batch["rm_scores"]
        assert rm.shape == (5, 5)
        # one non-zero at most per row, at the last valid response token
        valid = data.batch["attention_mask"][:, -5:].sum(-1)
        for i in range(5):
            nz = torch.nonzero(rm[i]).flatten().tolist()
            assert nz in ([], [int(valid[i]) - 1])
    finally:
        mgr.shutdown()
