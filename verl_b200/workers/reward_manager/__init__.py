"""Reward managers: turn (prompt, response, ground truth) rows into token-level score tensors.

Registry and classes follow verl/workers/reward_manager/{registry,abstract,naive,batch,dapo,prime}.py. The
scalar score of a sequence is written at its last valid response token.
"""

from __future__ import annotations

import asyncio
from abc import ABC, abstractmethod
from collections import defaultdict
from concurrent.futures import ProcessPoolExecutor
from typing import Any, Callable, Optional

import numpy as np
import torch

from ...protocol import DataProto
from ...utils.reward_score import default_compute_score

REWARD_MANAGER_REGISTRY: dict[str, type] = {}


def register(name: str):
    def deco(cls):
        if name in REWARD_MANAGER_REGISTRY and REWARD_MANAGER_REGISTRY[name] != cls:
            raise ValueError(f"Reward manager {name} has already been registered: {REWARD_MANAGER_REGISTRY[name]} vs {cls}")
        REWARD_MANAGER_REGISTRY[name] = cls
        return cls

    return deco


def get_reward_manager_cls(name: str):
    if name not in REWARD_MANAGER_REGISTRY:
        raise ValueError(f"Unknown reward manager: {name}")
    return REWARD_MANAGER_REGISTRY[name]


class AbstractRewardManager(ABC):
    @abstractmethod
    def __init__(self, tokenizer, num_examine: int, compute_score: Optional[Callable], reward_fn_key: str = "data_source",
                 **kwargs):
        ...

    @abstractmethod
    def __call__(self, data: DataProto, return_dict: bool = False):
        ...

    def _extract_reward_from_rm_scores(self, data: DataProto, return_dict: bool = False):
        if "rm_scores" not in data.batch.keys():
            return None
        if return_dict:
            keys = data.meta_info.get("reward_extra_keys", [])
            return {"reward_tensor": data.batch["rm_scores"],
                    "reward_extra_info": {k: data.non_tensor_batch[k] for k in keys}}
        return data.batch["rm_scores"]


def _decode(tokenizer, ids) -> str:
    if tokenizer is None:
        return " ".join(str(int(t)) for t in ids)
    return tokenizer.decode(ids, skip_special_tokens=True)


def _rows(data: DataProto, tokenizer):
    """Yield (i, prompt_str, response_str, valid_response_len, valid_response_ids) per sample."""
    P = data.batch["prompts"].shape[-1]
    for i in range(len(data)):
        mask = data.batch["attention_mask"][i]
        p_len = int(mask[:P].sum())
        r_len = int(mask[P:].sum())
        p_ids = data.batch["prompts"][i][P - p_len:] if p_len else data.batch["prompts"][i][:0]
        r_ids = data.batch["responses"][i][:r_len]
        yield i, _decode(tokenizer, p_ids), _decode(tokenizer, r_ids), r_len, r_ids


@register("naive")
class NaiveRewardManager(AbstractRewardManager):
    """One call of ``compute_score(data_source, solution_str, ground_truth, extra_info)`` per sample."""

    def __init__(self, tokenizer, num_examine: int = 0, compute_score=None, reward_fn_key: str = "data_source", **kwargs):
        self.tokenizer = tokenizer
        self.num_examine = num_examine
        self.compute_score = compute_score or default_compute_score
        self.reward_fn_key = reward_fn_key

    def __call__(self, data: DataProto, return_dict: bool = False):
        got = self._extract_reward_from_rm_scores(data, return_dict)
        if got is not None:
            return got
        reward = torch.zeros_like(data.batch["responses"], dtype=torch.float32)
        extra = defaultdict(list)
        printed: dict = {}
        for i, prompt, resp, r_len, r_ids in _rows(data, self.tokenizer):
            nt = {k: v[i] for k, v in data.non_tensor_batch.items()}
            gt = (nt.get("reward_model") or {}).get("ground_truth") if isinstance(nt.get("reward_model"), dict) else None
            source = nt.get(self.reward_fn_key, "unknown")
            info = nt.get("extra_info") or {}
            if isinstance(info, dict):
                info = dict(info)
                info.setdefault("num_turns", nt.get("__num_turns__"))
                info.setdefault("response_ids", r_ids)
            score = self.compute_score(data_source=source, solution_str=resp, ground_truth=gt, extra_info=info)
            if isinstance(score, dict):
                val = score["score"]
                for k, v in score.items():
                    extra[k].append(v)
            else:
                val = score
            if r_len > 0:
                reward[i, r_len - 1] = float(val)
            if printed.get(source, 0) < self.num_examine:
                printed[source] = printed.get(source, 0) + 1
                print("[prompt]", prompt, "\n[response]", resp, "\n[ground_truth]", gt, "\n[score]", score)
        if return_dict:
            return {"reward_tensor": reward, "reward_extra_info": dict(extra)}
        return reward


@register("batch")
class BatchRewardManager(AbstractRewardManager):
    """Scores the whole batch in one call: ``compute_score(data_sources=, solution_strs=, ground_truths=, extra_infos=)``."""

    def __init__(self, tokenizer, num_examine: int = 0, compute_score=None, reward_fn_key: str = "data_source",
                 **reward_kwargs):
        self.tokenizer = tokenizer
        self.num_examine = num_examine
        self.compute_score = compute_score
        self.reward_fn_key = reward_fn_key
        self.reward_kwargs = reward_kwargs

    def __call__(self, data: DataProto, return_dict: bool = False):
        got = self._extract_reward_from_rm_scores(data, return_dict)
        if got is not None:
            return got
        rows = list(_rows(data, self.tokenizer))
        n = len(rows)
        gts = [(data.non_tensor_batch["reward_model"][i] or {}).get("ground_truth") for i in range(n)]
        sources = list(data.non_tensor_batch[self.reward_fn_key])
        infos = list(data.non_tensor_batch.get("extra_info", [None] * n))
        scores = self.compute_score(data_sources=sources, solution_strs=[r[2] for r in rows], ground_truths=gts,
                                    extra_infos=infos, **self.reward_kwargs)
        reward = torch.zeros_like(data.batch["responses"], dtype=torch.float32)
        extra = defaultdict(list)
        for (i, _, _, r_len, _), sc in zip(rows, scores):
            if isinstance(sc, dict):
                val = sc["score"]
                for k, v in sc.items():
                    extra[k].append(v)
            else:
                val = sc
            if r_len > 0:
                reward[i, r_len - 1] = float(val)
        if return_dict:
            return {"reward_tensor": reward, "reward_extra_info": dict(extra)}
        return reward


@register("dapo")
class DAPORewardManager(NaiveRewardManager):
    """Naive scoring plus the soft overlong penalty of DAPO: responses longer than
    ``max_resp_len - overlong_buffer.len`` lose up to ``penalty_factor``, linearly."""

    def __init__(self, tokenizer, num_examine: int = 0, compute_score=None, reward_fn_key: str = "data_source",
                 max_resp_len: Optional[int] = None, overlong_buffer_cfg=None, **kwargs):
        super().__init__(tokenizer, num_examine, compute_score, reward_fn_key)
        self.max_resp_len = max_resp_len
        self.overlong_buffer_cfg = overlong_buffer_cfg
        if overlong_buffer_cfg is not None:
            assert max_resp_len is not None, f"max_resp_len must be provided if {overlong_buffer_cfg=}, but got None"
            assert max_resp_len >= overlong_buffer_cfg["len"], "max_resp_len must be larger than overlong_buffer.len"

    def __call__(self, data: DataProto, return_dict: bool = False):
        out = super().__call__(data, return_dict=True)
        if "rm_scores" in data.batch.keys():
            return out if return_dict else out["reward_tensor"]
        reward, extra = out["reward_tensor"], out["reward_extra_info"]
        cfg = self.overlong_buffer_cfg
        if cfg is not None and cfg.get("enable", False):
            P = data.batch["prompts"].shape[-1]
            lens = data.batch["attention_mask"][:, P:].sum(-1)
            expected = self.max_resp_len - cfg["len"]
            pen = torch.clamp(-(lens - expected).float() / cfg["len"] * cfg["penalty_factor"], max=0.0)
            for i in range(len(data)):
                if lens[i] > 0:
                    reward[i, int(lens[i]) - 1] += pen[i]
            if cfg.get("log", False):
                extra["overlong_reward"] = pen.tolist()
                extra["overlong"] = (pen < 0).tolist()
        if return_dict:
            return {"reward_tensor": reward, "reward_extra_info": extra}
        return reward


def _score_one(args):
    fn, source, resp, gt, info = args
    try:
        return fn(data_source=source, solution_str=resp, ground_truth=gt, extra_info=info)
    except Exception:
        return 0.0


@register("prime")
class PrimeRewardManager(NaiveRewardManager):
    """Scores samples in a process pool with a per-sample time-out (slow verifiers such as code / math checkers)."""

    def __init__(self, tokenizer, num_examine: int = 0, compute_score=None, reward_fn_key: str = "data_source",
                 num_processes: int = 8, timeout: float = 300.0, **kwargs):
        super().__init__(tokenizer, num_examine, compute_score, reward_fn_key)
        self.num_processes, self.timeout = num_processes, timeout

    def __call__(self, data: DataProto, return_dict: bool = False):
        got = self._extract_reward_from_rm_scores(data, return_dict)
        if got is not None:
            return got
        rows = list(_rows(data, self.tokenizer))
        jobs = []
        for i, _, resp, _, _ in rows:
            rm = data.non_tensor_batch["reward_model"][i] or {}
            jobs.append((self.compute_score, data.non_tensor_batch[self.reward_fn_key][i], resp, rm.get("ground_truth"),
                         data.non_tensor_batch.get("extra_info", [None] * len(rows))[i]))
        scores = [0.0] * len(jobs)
        with ProcessPoolExecutor(max_workers=self.num_processes) as ex:
            futs = [ex.submit(_score_one, j) for j in jobs]
            for k, f in enumerate(futs):
                try:
                    scores[k] = f.result(timeout=self.timeout)
                except Exception:
                    scores[k] = 0.0
        reward = torch.zeros_like(data.batch["responses"], dtype=torch.float32)
        for (i, _, _, r_len, _), sc in zip(rows, scores):
            val = sc["score"] if isinstance(sc, dict) else sc
            if r_len > 0:
                reward[i, r_len - 1] = float(val)
        if return_dict:
            return {"reward_tensor": reward, "reward_extra_info": {}}
        return reward


__all__ = ["register", "get_reward_manager_cls", "AbstractRewardManager", "NaiveRewardManager", "BatchRewardManager",
           "DAPORewardManager", "PrimeRewardManager"]
