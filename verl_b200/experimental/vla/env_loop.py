"""Pipelined environment / policy stages for embodied rollouts.

Role of verl/experimental/vla/ (``EnvWorker :72``, ``EnvLoop :30``, ``NaiveRolloutRob :112``): environments are split
in ``stage_num`` groups; while the policy computes actions for one group the simulator steps another, so neither
side idles. Actions are discretised into ``n_action_bins`` tokens per dimension (the OpenVLA action tokenisation) so
that the trajectory is a token sequence the PPO machinery can train on: per step the batch gets ``responses`` (action
tokens), ``old_log_probs`` and the environment reward; ``to_dataproto`` lays the finished trajectories out as
[prompt | response] rows with a response mask.

Any callable ``policy(obs) -> (action_tokens, log_probs)`` drives the loop:
``verl_b200.models.openvla_oft.OpenVLAPolicy`` wraps the OpenVLA-OFT vision-language-action model (images + task
string in, one parallel-decoded action chunk out), ``NaiveRolloutRob`` wraps a token-level language model that reads a
tokenised state. The reference's simulators (LIBERO, Isaac) need a graphics stack; ``envs/synthetic_env.py`` has the
same interface without one.
"""

from __future__ import annotations

import concurrent.futures as cf
from dataclasses import dataclass, field
from typing import Callable, Optional

import numpy as np
import torch

from ...protocol import DataProto


class ActionTokenizer:
    def __init__(self, n_bins: int = 256, low: float = -1.0, high: float = 1.0, vocab_offset: int = 0):
        self.n_bins, self.low, self.high, self.vocab_offset = n_bins, low, high, vocab_offset
        self.centers = (np.linspace(low, high, n_bins + 1)[:-1] + np.linspace(low, high, n_bins + 1)[1:]) / 2

    def encode(self, actions: np.ndarray) -> np.ndarray:
        x = np.clip(actions, self.low, self.high)
        return (np.minimum(((x - self.low) / (self.high - self.low) * self.n_bins).astype(np.int64), self.n_bins - 1)
                + self.vocab_offset)

    def decode(self, tokens: np.ndarray) -> np.ndarray:
        return self.centers[np.clip(np.asarray(tokens) - self.vocab_offset, 0, self.n_bins - 1)].astype(np.float32)


class EnvWorker:
    """Owns one group of environments; ``step`` runs in a worker thread so that it overlaps the policy."""

    def __init__(self, env_fn: Callable[[], object]):
        self.env = env_fn()
        self._pool = cf.ThreadPoolExecutor(max_workers=1)
        self.obs = None

    def reset(self):
        self.obs = self.env.reset()
        return self.obs

    def step_async(self, actions: np.ndarray) -> cf.Future:
        return self._pool.submit(self.env.step, actions)

    def close(self):
        self._pool.shutdown(wait=True)


@dataclass
class Trajectory:
    states: list = field(default_factory=list)
    tokens: list = field(default_factory=list)
    logps: list = field(default_factory=list)
    rewards: list = field(default_factory=list)
    alive: list = field(default_factory=list)


class EnvLoop:
    def __init__(self, env_fns: list[Callable[[], object]], policy: Callable, action_tokenizer: Optional[ActionTokenizer] = None,
                 max_steps: int = 16):
        self.workers = [EnvWorker(fn) for fn in env_fns]  # one worker per pipeline stage
        self.policy = policy
        self.tok = action_tokenizer or ActionTokenizer()
        self.max_steps = max_steps

    def run(self) -> list[Trajectory]:
        trajs = [Trajectory() for _ in self.workers]
        obs = [w.reset() for w in self.workers]
        alive = [np.ones(w.env.num_envs, bool) for w in self.workers]
        pending: list[Optional[cf.Future]] = [None] * len(self.workers)
        for _ in range(self.max_steps):
            for s, w in enumerate(self.workers):
                if pending[s] is not None:  # the simulator stepped this stage while the policy served the others
                    obs[s], r, term, trunc, _ = pending[s].result()
                    trajs[s].rewards.append(r)
                    alive[s] = alive[s] & ~(term | trunc)
                    pending[s] = None
                if not alive[s].any():
                    continue
                tokens, logp = self.policy(obs[s])
                trajs[s].states.append(obs[s]["state"].copy())
                trajs[s].tokens.append(np.asarray(tokens))
                trajs[s].logps.append(np.asarray(logp, np.float32))
                trajs[s].alive.append(alive[s].copy())
                pending[s] = w.step_async(self.tok.decode(np.asarray(tokens)))
        for s, f in enumerate(pending):
            if f is not None:
                _, r, _, _, _ = f.result()
                trajs[s].rewards.append(r)
        return trajs

    def close(self):
        for w in self.workers:
            w.close()

    def to_dataproto(self, trajs: list[Trajectory], prompt_len: int = 1, pad_id: int = 0) -> DataProto:
        """One row per environment: response = all action tokens of the episode, score on its last live token."""
        rows_tok, rows_lp, rows_mask, scores = [], [], [], []
        A = None
        for tr in trajs:
            if not tr.tokens:
                continue
            toks = np.stack(tr.tokens, 1)          # [E, steps, A]
            lps = np.stack(tr.logps, 1)
            live = np.stack(tr.alive, 1)           # [E, steps]
            rew = np.stack(tr.rewards, 1) if tr.rewards else np.zeros(live.shape, np.float32)
            E, S, A = toks.shape
            rows_tok.append(toks.reshape(E, S * A))
            rows_lp.append(lps.reshape(E, S * A))
            rows_mask.append(np.repeat(live, A, axis=1))
            scores.append(rew[:, : live.shape[1]].sum(1))
        R = self.max_steps * (A or 1)

        def pad(x, value):
            out = np.full((x.shape[0], R), value, x.dtype)
            out[:, : x.shape[1]] = x
            return out

        resp = torch.from_numpy(np.concatenate([pad(t, pad_id) for t in rows_tok]))
        mask = torch.from_numpy(np.concatenate([pad(m.astype(np.int64), 0) for m in rows_mask]))
        lp = torch.from_numpy(np.concatenate([pad(l, 0.0) for l in rows_lp]))
        score = torch.from_numpy(np.concatenate(scores)).float()
        B = resp.shape[0]
        prompts = torch.full((B, prompt_len), pad_id, dtype=torch.long)
        tls = torch.zeros(B, R)
        last = (mask.sum(-1) - 1).clamp(min=0)
        tls[torch.arange(B), last] = score
        attn = torch.cat([torch.ones(B, prompt_len, dtype=torch.long), mask], 1)
        return DataProto.from_dict(tensors={"prompts": prompts, "responses": resp, "response_mask": mask, "attention_mask": attn,
                                            "input_ids": torch.cat([prompts, resp], 1), "rollout_log_probs": lp,
                                            "token_level_scores": tls})


class NaiveRolloutRob:
    """Token-level policy adapter: the state is discretised into tokens, a causal LM (``model(batch)`` returning logits
    for packed tokens) emits ``action_dim`` action tokens one after the other."""

    def __init__(self, model, action_dim: int, n_bins: int = 256, temperature: float = 1.0, seed: int = 0):
        self.model, self.action_dim, self.n_bins, self.temperature = model, action_dim, n_bins, temperature
        self.state_tok = ActionTokenizer(n_bins)
        self.gen = torch.Generator().manual_seed(seed)

    @torch.no_grad()
    def __call__(self, obs: dict):
        from ...models.transformer import PackedBatch

        state = self.state_tok.encode(obs["state"])  # [E, S]
        E, S = state.shape
        seq = torch.from_numpy(state)
        toks, lps = [], []
        for _ in range(self.action_dim):
            L = seq.shape[1]
            batch = PackedBatch(seq.reshape(-1), torch.arange(L).repeat(E), torch.arange(0, E * L + 1, L, dtype=torch.int32), L)
            hidden = self.model.forward_hidden(batch)[L - 1 :: L]
            logits = self.model.logits(hidden).float()[:, : self.n_bins] / max(self.temperature, 1e-6)
            logp = torch.log_softmax(logits, -1)
            a = torch.multinomial(logp.exp(), 1, generator=self.gen)[:, 0]
            toks.append(a)
            lps.append(logp.gather(1, a[:, None])[:, 0])
            seq = torch.cat([seq, a[:, None]], 1)
        return torch.stack(toks, 1).numpy(), torch.stack(lps, 1).numpy()
