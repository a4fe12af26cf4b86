"""RoboCasa task wrapper (reference ``src/opentau/envs/robocasa.py:98-985``).

As with LIBERO the simulator comes from a backend (``make(task, split, seed, cameras, height, width) -> sim`` with
``reset() -> obs``, ``step(action_dict) -> (obs, reward, done, info)``, ``check_success()``, ``language``, ``close()``);
``real_backend()`` builds it on the installed ``robocasa`` package and needs its kitchen assets and a graphics context.
Kept from the reference: the flat 12-D action split into the simulator's action dict (base motion 4, control mode 1,
end-effector position 3, rotation 3, gripper 1), camera images mapped to ``camera{k}``, a 16-D proprioceptive state
(base position 3, base rotation 4, end-effector position 3, rotation 4, gripper 2; missing parts read zero), and the
official per-task horizons with a default.
"""

from __future__ import annotations

from typing import Any, Sequence

import numpy as np

from ..utils.io_utils import silence_output_unless_error

ACTION_DIM, STATE_DIM = 12, 16
DEFAULT_HORIZON = 500
OFFICIAL_HORIZONS = {"NavigateKitchen": 500, "CloseSingleDoor": 500, "OpenSingleDoor": 500, "CloseDrawer": 500,
                     "OpenDrawer": 500, "TurnOnMicrowave": 500, "TurnOffMicrowave": 500, "PnPCounterToCab": 500,
                     "PnPCabToCounter": 500, "CoffeePressButton": 300, "TurnOnSinkFaucet": 500, "TurnOffSinkFaucet": 500}
STATE_PARTS = (("robot0_base_pos", 3), ("robot0_base_quat", 4), ("robot0_eef_pos", 3), ("robot0_eef_quat", 4),
               ("robot0_gripper_qpos", 2))


def convert_action(flat_action) -> dict[str, np.ndarray]:
    a = np.asarray(flat_action, np.float32)
    if a.shape[-1] < ACTION_DIM:
        raise ValueError(f"RoboCasa actions have {ACTION_DIM} values, got {a.shape[-1]}")
    return {"action.base_motion": a[0:4], "action.control_mode": a[4:5], "action.end_effector_position": a[5:8],
            "action.end_effector_rotation": a[8:11], "action.gripper_close": a[11:12]}


def parse_camera_names(camera_name: str | Sequence[str]) -> list[str]:
    names = [c.strip() for c in camera_name.split(",")] if isinstance(camera_name, str) else list(camera_name)
    if not [c for c in names if c]:
        raise ValueError("camera_name resolved to an empty list")
    return [c for c in names if c]


def official_task_horizon(task: str) -> int:
    return OFFICIAL_HORIZONS.get(task, DEFAULT_HORIZON)


def resolve_tasks(task: str) -> list[str]:
    """Comma-separated task names; duplicates removed, order kept."""
    seen, out = set(), []
    for t in (x.strip() for x in task.split(",")):
        if t and t not in seen:
            seen.add(t)
            out.append(t)
    if not out:
        raise ValueError("no RoboCasa task given")
    return out


class RoboCasaEnv:
    def __init__(self, backend, task: str, camera_names: Sequence[str], observation_height: int = 256,
                 observation_width: int = 256, split: str = "pretrain", episode_length: int | None = None):
        self.task, self.split = task, split
        self.camera_names = parse_camera_names(camera_names)
        self._backend, self._hw = backend, (observation_height, observation_width)
        self._max_episode_steps = episode_length or official_task_horizon(task)
        self._env, self.task_description, self._steps = None, task, 0

    def _format(self, raw: dict[str, Any]) -> dict[str, Any]:
        images = {f"camera{k}": np.asarray(raw[f"{cam}_image"]) for k, cam in enumerate(self.camera_names)}
        state = np.concatenate([np.asarray(raw.get(key, np.zeros(n)), np.float64).reshape(-1)[:n]
                                for key, n in STATE_PARTS])
        return {"pixels": images, "agent_pos": state}

    def reset(self, seed: int | None = None, options: dict | None = None):
        if self._env is not None:
            self._env.close()
        self._env = self._backend.make(self.task, self.split, seed, self.camera_names, *self._hw)
        raw = self._env.reset()
        self.task_description = getattr(self._env, "language", None) or self.task
        self._steps = 0
        return self._format(raw), {"is_success": False}

    def step(self, action):
        raw, reward, done, info = self._env.step(convert_action(action))
        self._steps += 1
        success = bool(self._env.check_success())
        truncated = self._steps >= self._max_episode_steps and not success
        return self._format(raw), float(reward), bool(done or success), truncated, dict(info or {}, is_success=success)

    def render(self) -> np.ndarray:
        raise RuntimeError("rendering needs the simulator's own viewer")

    def close(self) -> None:
        if self._env is not None:
            self._env.close()
            self._env = None


def real_backend():  # pragma: no cover - needs the simulator, its assets and a graphics context
    import robocasa  # noqa: F401
    import robosuite

    class Backend:
        def make(self, task, split, seed, cameras, height, width):
            with silence_output_unless_error(label=f"robocasa task={task} split={split}"):
                env = robosuite.make(env_name=task, robots="PandaOmron", has_renderer=False,
                                     has_offscreen_renderer=True, use_camera_obs=True, camera_names=list(cameras),
                                     camera_heights=height, camera_widths=width, seed=seed, obj_instance_split=split)
            env.language = env.get_ep_meta().get("lang", task)
            inner_step = env.step

            def step(action_dict):
                flat = np.concatenate([action_dict[k] for k in ("action.end_effector_position",
                                                                "action.end_effector_rotation", "action.gripper_close",
                                                                "action.base_motion", "action.control_mode")])
                return inner_step(flat)
            env.step = step
            env.check_success = env._check_success
            return env

    return Backend()


def create_robocasa_envs(cfg, n_envs: int, backend=None) -> dict[str, dict[int, Any]]:
    from .fake import SyncVectorEnv
    backend = backend or real_backend()
    out: dict[str, dict[int, Any]] = {}
    for i, task in enumerate(resolve_tasks(cfg.task or "")):
        fns = [lambda task=task: RoboCasaEnv(backend, task, cfg.camera_names, episode_length=cfg.episode_length)
               for _ in range(n_envs)]
        out[task] = {i: SyncVectorEnv(fns)}
    return out
