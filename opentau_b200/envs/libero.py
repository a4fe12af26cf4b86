"""LIBERO task wrapper (reference ``src/opentau/envs/libero.py:39-447``, ``utils/libero.py:31-214``).

The simulator (``libero`` + robosuite + MuJoCo) renders through OpenGL / EGL and is not present on a headless CUDA box,
so the wrapper takes its simulator from a *backend*: an object with ``get_task(task_suite_name, task_id) -> (name,
language, init_states | None)`` and ``make(task_suite_name, task_id, height, width, control_freq) -> sim`` where ``sim``
has the ``OffScreenRenderEnv`` surface (``seed, set_init_state, reset, step, check_success, close``).  ``real_backend()``
builds that from the installed ``libero`` package and raises ImportError without it; tests inject a fake one.  Everything
else is the reference's behaviour: both cameras rotated by 180 degrees and mapped to ``camera0 / camera1``, an 8-D state
(end-effector position, axis-angle orientation, gripper opening), 7-D actions in [-1, 1] (longer vectors are cut), ten
no-op steps after every reset, success = the simulator's own check, per-suite step limits.
"""

from __future__ import annotations

import math
from typing import Any, Iterable, Sequence

import numpy as np

from ..utils.io_utils import silence_output_unless_error

OBS_STATE_DIM, ACTION_DIM = 8, 7
TASK_SUITE_MAX_STEPS = {"libero_spatial": 280, "libero_object": 280, "libero_goal": 300, "libero_10": 520,
                        "libero_90": 400}
DEFAULT_CAMERA_MAPPING = {"agentview_image": ["camera0"], "robot0_eye_in_hand_image": ["camera1"]}


def get_libero_dummy_action() -> list[float]:
    """No-op used to let the scene settle: zero motion, gripper open."""
    return [0, 0, 0, 0, 0, 0, -1]


def parse_camera_names(camera_name: str | Sequence[str]) -> list[str]:
    names = [c.strip() for c in camera_name.split(",")] if isinstance(camera_name, str) else list(camera_name)
    names = [c for c in names if c]
    if not names:
        raise ValueError("camera_name resolved to an empty list")
    return names


def select_task_ids(total_tasks: int, task_ids: Iterable[int] | None) -> list[int]:
    if task_ids is None:
        return list(range(total_tasks))
    ids = sorted({int(t) for t in task_ids})
    bad = [t for t in ids if t < 0 or t >= total_tasks]
    if bad:
        raise ValueError(f"task ids {bad} out of range for a suite of {total_tasks} tasks")
    return ids


def quat2axisangle(quat) -> np.ndarray:
    """(x, y, z, w) -> axis * angle; zero for the identity."""
    q = np.asarray(quat, np.float64).copy()
    q[3] = np.clip(q[3], -1.0, 1.0)
    den = math.sqrt(1.0 - q[3] * q[3])
    if math.isclose(den, 0.0):
        return np.zeros(3)
    return q[:3] * 2.0 * math.acos(q[3]) / den


def summarize_libero_results(results: list[int]) -> dict:
    """``results``: steps to success (>= 0), -1 failure, -2 crash."""
    if not results:
        return {"message": "No results to summarize."}
    ok = [i for i, r in enumerate(results) if r >= 0]
    fail = [i for i, r in enumerate(results) if r == -1]
    crash = [i for i, r in enumerate(results) if r == -2]
    n = len(results)
    return {"total_simulations": n, "success_indices": ok, "failure_indices": fail, "crashed_indices": crash,
            "success_count": len(ok), "failure_count": len(fail), "crashed_count": len(crash),
            "success_rate": len(ok) / n, "failure_rate": len(fail) / n, "crashed_rate": len(crash) / n,
            "steps_taken": results,
            "avg_steps_taken_until_success": float(np.mean([results[i] for i in ok])) if ok else None}


class LiberoEnv:
    metadata = {"render_modes": ["rgb_array"], "render_fps": 80}

    def __init__(self, backend, task_suite_name: str, task_id: int, camera_name="agentview_image,robot0_eye_in_hand_image",
                 obs_type: str = "pixels_agent_pos", observation_width: int = 256, observation_height: int = 256,
                 init_states: bool = True, episode_index: int = 0, camera_name_mapping: dict[str, list[str]] | None = None,
                 num_steps_wait: int = 10, control_freq: int = 20):
        if obs_type not in ("pixels", "pixels_agent_pos"):
            raise NotImplementedError(f"observation type {obs_type!r} is not supported (use 'pixels' or 'pixels_agent_pos')")
        self.task_id, self.obs_type = task_id, obs_type
        self.camera_name = parse_camera_names(camera_name)
        self.camera_name_mapping = camera_name_mapping or dict(DEFAULT_CAMERA_MAPPING)
        for cam, to in self.camera_name_mapping.items():
            if isinstance(to, str):
                raise TypeError(f"camera_name_mapping[{cam!r}] must be a list of names, got the string {to!r}")
        self.num_steps_wait = num_steps_wait
        self.task, self.task_description, states = backend.get_task(task_suite_name, task_id)
        self._init_states = states if init_states else None
        self._init_state_id = episode_index
        self._env = backend.make(task_suite_name, task_id, observation_height, observation_width, control_freq)
        self._max_episode_steps = TASK_SUITE_MAX_STEPS.get(task_suite_name, 500)

    def _format_raw_obs(self, raw: dict[str, Any]) -> dict[str, Any]:
        images = {}
        for cam in self.camera_name:
            img = raw[cam][::-1, ::-1]                       # the simulator's cameras are upside down
            for name in self.camera_name_mapping[cam]:
                images[name] = img.copy()
        if self.obs_type == "pixels":
            return {"pixels": images}
        state = np.concatenate([raw["robot0_eef_pos"], quat2axisangle(raw["robot0_eef_quat"]), raw["robot0_gripper_qpos"]])
        return {"pixels": images, "agent_pos": state}

    def reset(self, seed: int | None = None, options: dict | None = None):
        self._env.seed(seed)
        if self._init_states is not None:
            self._env.set_init_state(self._init_states[self._init_state_id % len(self._init_states)])
        raw = self._env.reset()
        for _ in range(self.num_steps_wait):
            raw, _, _, _ = self._env.step(get_libero_dummy_action())
        return self._format_raw_obs(raw), {"is_success": False}

    def step(self, action):
        action = np.asarray(action)
        if action.ndim != 1:
            raise ValueError(f"expected a 1-D action, got shape {action.shape}")
        raw, reward, done, info = self._env.step(action[:ACTION_DIM])
        success = bool(self._env.check_success())
        info = dict(info or {}, is_success=success)
        obs = self._format_raw_obs(raw)
        if done:
            self.reset()
            info.update(task=self.task, task_id=self.task_id, done=done)
        return obs, float(reward), bool(done or success), False, info

    def render(self) -> np.ndarray:
        cams = self._format_raw_obs(self._env.env._get_observations())["pixels"]
        return np.concatenate(list(cams.values()), axis=1)

    def close(self) -> None:
        self._env.close()


def real_backend():  # pragma: no cover - needs the simulator and a graphics context
    """Backend on the installed ``libero`` package."""
    import os

    from libero.libero import benchmark, get_libero_path
    from libero.libero.envs import OffScreenRenderEnv

    class Backend:
        def _suite(self, name):
            suites = benchmark.get_benchmark_dict()
            if name not in suites:
                raise ValueError(f"unknown LIBERO suite {name!r}; available: {sorted(suites)}")
            return suites[name]()

        def num_tasks(self, name):
            return len(self._suite(name).tasks)

        def get_task(self, name, task_id):
            suite = self._suite(name)
            task = suite.get_task(task_id)
            return task.name, task.language, suite.get_task_init_states(task_id)

        def make(self, name, task_id, height, width, control_freq):
            task = self._suite(name).get_task(task_id)
            # the simulator prints a banner per worker; it is shown only when construction fails
            with silence_output_unless_error(label=f"libero suite={name} task={task_id}"):
                env = OffScreenRenderEnv(bddl_file_name=os.path.join(get_libero_path("bddl_files"),
                                                                     task.problem_folder, task.bddl_file),
                                         camera_heights=height, camera_widths=width, control_freq=control_freq)
                env.reset()
            return env

    return Backend()


def create_libero_envs(cfg, n_envs: int, backend=None) -> dict[str, dict[int, Any]]:
    """``{suite: {task_id: vector env of n_envs copies}}``; copy ``i`` starts from initial state ``i``."""
    from .fake import SyncVectorEnv
    backend = backend or real_backend()
    out: dict[str, dict[int, Any]] = {}
    for suite in [s.strip() for s in (cfg.task or "").split(",") if s.strip()]:
        ids = select_task_ids(backend.num_tasks(suite), cfg.task_ids)
        out[suite] = {}
        for tid in ids:
            fns = [lambda tid=tid, i=i: LiberoEnv(backend, suite, tid, cfg.camera_name, "pixels_agent_pos",
                                                  cfg.observation_width, cfg.observation_height, cfg.init_states, i)
                   for i in range(n_envs)]
            out[suite][tid] = SyncVectorEnv(fns)
    return out
