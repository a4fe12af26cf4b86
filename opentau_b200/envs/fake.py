"""Headless stand-in for the simulated robots, with the gymnasium calling convention
(``reset(seed) -> (obs, info)``, ``step(a) -> (obs, reward, terminated, truncated, info)``) and a synchronous
vector wrapper with auto-reset bookkeeping like ``gymnasium.vector`` (``final_info`` / ``is_success``).

Dynamics: a point in ``[-1,1]^action_dim`` moves by ``action_scale * clip(action, -1, 1)``; the goal is drawn at
reset.  ``agent_pos = [position | goal | 0...]``.  The camera image is rendered on the CPU with numpy (a dot for the
agent, a cross for the goal), so observation pipelines see real pixel arrays.
"""

from __future__ import annotations

from typing import Any, Callable

import numpy as np


class FakeRobotEnv:
    metadata = {"render_fps": 30}

    def __init__(self, task: str = "reach the goal", state_dim: int = 8, action_dim: int = 4, num_cams: int = 1,
                 resolution: tuple[int, int] = (64, 64), tolerance: float = 0.1, action_scale: float = 0.25,
                 episode_length: int = 40, task_id: int = 0):
        if state_dim < 2 * action_dim:
            raise ValueError("state_dim must hold position and goal (>= 2 * action_dim)")
        self.task, self.task_id = task, task_id
        self.state_dim, self.action_dim, self.num_cams = state_dim, action_dim, num_cams
        self.resolution, self.tolerance, self.action_scale = tuple(resolution), tolerance, action_scale
        self._max_episode_steps = episode_length
        self.rng = np.random.default_rng(0)
        self.pos = np.zeros(action_dim, np.float32)
        self.goal = np.zeros(action_dim, np.float32)
        self.t = 0

    def task_description(self) -> str:
        return self.task

    def _render(self) -> np.ndarray:
        H, W = self.resolution
        img = np.full((H, W, 3), 32, np.uint8)

        def px(p):
            return (int((p[1] * 0.5 + 0.5) * (H - 1)), int((p[0] * 0.5 + 0.5) * (W - 1)))

        gy, gx = px(self.goal)
        img[max(0, gy - 3):gy + 4, gx] = (0, 255, 0)
        img[gy, max(0, gx - 3):gx + 4] = (0, 255, 0)
        ay, ax = px(self.pos)
        img[max(0, ay - 1):ay + 2, max(0, ax - 1):ax + 2] = (255, 64, 64)
        return img

    def _obs(self) -> dict[str, Any]:
        st = np.zeros(self.state_dim, np.float32)
        st[:self.action_dim], st[self.action_dim:2 * self.action_dim] = self.pos, self.goal
        img = self._render()
        return {"agent_pos": st, "pixels": {f"camera{i}": img for i in range(self.num_cams)}}

    def reset(self, seed: int | None = None, options: dict | None = None):
        if seed is not None:
            self.rng = np.random.default_rng(seed)
        self.pos = self.rng.uniform(-0.5, 0.5, self.action_dim).astype(np.float32)
        self.goal = self.rng.uniform(-0.8, 0.8, self.action_dim).astype(np.float32)
        self.t = 0
        return self._obs(), {"is_success": False, "task": self.task}

    def step(self, action):
        a = np.clip(np.asarray(action, np.float32)[:self.action_dim], -1.0, 1.0)
        self.pos = np.clip(self.pos + self.action_scale * a, -1.0, 1.0)
        self.t += 1
        dist = float(np.linalg.norm(self.pos - self.goal))
        success = dist < self.tolerance
        truncated = self.t >= self._max_episode_steps
        return self._obs(), -dist, bool(success), bool(truncated), {"is_success": bool(success), "task": self.task}

    def render(self) -> np.ndarray:
        return self._render()

    def close(self) -> None:
        pass


def _stack(obs_list: list[dict]) -> dict:
    out: dict[str, Any] = {}
    for k, v in obs_list[0].items():
        out[k] = _stack([o[k] for o in obs_list]) if isinstance(v, dict) else np.stack([o[k] for o in obs_list])
    return out


class SyncVectorEnv:
    """Steps ``n`` environments in lock step; a finished environment is reset on the spot and its last step's info
    is reported under ``final_info`` (the convention the rollout loop relies on)."""

    def __init__(self, env_fns: list[Callable[[], FakeRobotEnv]]):
        self.envs = [fn() for fn in env_fns]
        self.num_envs = len(self.envs)

    def call(self, name: str, *args):
        vals = []
        for e in self.envs:
            attr = getattr(e, name)
            vals.append(attr(*args) if callable(attr) else attr)
        return tuple(vals)

    def reset(self, seed: int | list[int] | None = None):
        seeds = seed if isinstance(seed, (list, tuple)) else [None if seed is None else seed + i for i in range(self.num_envs)]
        res = [e.reset(seed=s) for e, s in zip(self.envs, seeds)]
        return _stack([r[0] for r in res]), {"is_success": np.array([False] * self.num_envs)}

    def step(self, actions):
        obs, rew, term, trunc, infos = [], [], [], [], []
        final: list[dict | None] = [None] * self.num_envs
        for i, (e, a) in enumerate(zip(self.envs, np.asarray(actions))):
            o, r, te, tr, info = e.step(a)
            if te or tr:
                final[i] = info
                o, _ = e.reset()
            obs.append(o), rew.append(r), term.append(te), trunc.append(tr), infos.append(info)
        info = {"is_success": np.array([i["is_success"] for i in infos])}
        if any(f is not None for f in final):
            info["final_info"] = final
        return _stack(obs), np.asarray(rew, np.float32), np.asarray(term), np.asarray(trunc), info

    def close(self) -> None:
        for e in self.envs:
            e.close()
