"""A vectorised toy manipulation task that needs no simulator and no graphics stack.

The reference trains OpenVLA-OFT policies in LIBERO (MuJoCo off-screen rendering) and Isaac Sim
(verl/experimental/vla/envs/); both need a graphics stack. This environment has the same interface the env workers
use (``reset`` / ``step`` on a batch of environments, image observations, a language instruction, sparse success
reward) with observations rasterised by numpy: a 2-D reach task, the arm tip and the target drawn as squares into a
small RGB image.
"""

from __future__ import annotations

import numpy as np


class SyntheticReachEnv:
    def __init__(self, num_envs: int, image_size: int = 32, max_steps: int = 16, action_dim: int = 2, seed: int = 0,
                 success_radius: float = 0.12):
        self.num_envs, self.image_size, self.max_steps, self.action_dim = num_envs, image_size, max_steps, action_dim
        self.success_radius = success_radius
        self.rng = np.random.default_rng(seed)
        self.pos = np.zeros((num_envs, 2), np.float32)
        self.goal = np.zeros((num_envs, 2), np.float32)
        self.t = np.zeros(num_envs, np.int32)
        self.done = np.zeros(num_envs, bool)

    def task_descriptions(self) -> list[str]:
        return ["move the red square onto the green square"] * self.num_envs

    def reset(self, env_ids=None):
        ids = np.arange(self.num_envs) if env_ids is None else np.asarray(env_ids)
        self.pos[ids] = self.rng.uniform(-1, 1, (len(ids), 2))
        self.goal[ids] = self.rng.uniform(-1, 1, (len(ids), 2))
        self.t[ids] = 0
        self.done[ids] = False
        return self._obs()

    def _draw(self, img, xy, channel):
        s = self.image_size
        c = np.clip(((xy + 1) / 2 * (s - 1)).astype(int), 1, s - 2)
        for e in range(self.num_envs):
            img[e, c[e, 1] - 1 : c[e, 1] + 2, c[e, 0] - 1 : c[e, 0] + 2, channel] = 255

    def _obs(self) -> dict:
        img = np.zeros((self.num_envs, self.image_size, self.image_size, 3), np.uint8)
        self._draw(img, self.pos, 0)
        self._draw(img, self.goal, 1)
        return {"images": img, "state": np.concatenate([self.pos, self.goal], -1), "task": self.task_descriptions()}

    def step(self, actions: np.ndarray):
        """actions [num_envs, action_dim] in [-1, 1]. Returns (obs, reward, terminated, truncated, info)."""
        a = np.clip(np.asarray(actions, np.float32)[:, :2], -1, 1) * 0.25
        live = ~self.done
        self.pos[live] = np.clip(self.pos[live] + a[live], -1, 1)
        self.t[live] += 1
        dist = np.linalg.norm(self.pos - self.goal, axis=-1)
        success = (dist < self.success_radius) & live
        truncated = (self.t >= self.max_steps) & live & ~success
        reward = success.astype(np.float32)
        self.done |= success | truncated
        return self._obs(), reward, success, truncated, {"distance": dist, "success": success}

    @staticmethod
    def expert_action(state: np.ndarray) -> np.ndarray:
        d = state[:, 2:4] - state[:, 0:2]
        return np.clip(d / 0.25, -1, 1)
