"""LIBERO / RoboCasa wrappers against scripted simulator backends (the real simulators need a graphics context)."""

import numpy as np
import pytest
import torch

from opentau_b200.envs import libero, robocasa
from opentau_b200.envs.configs import LiberoEnvConfig, RoboCasaEnvConfig
from opentau_b200.envs.factory import make_envs
from opentau_b200.scripts.eval import eval_policy


class _LiberoSim:
    """Gripper position integrates the first three action values; success when x > 0.5."""

    def __init__(self, h, w):
        self.h, self.w, self.pos, self.init, self.seeded = h, w, np.zeros(3), None, None
        self.env = self

    def seed(self, s):
        self.seeded = s

    def set_init_state(self, st):
        self.init = np.asarray(st, float)

    def _get_observations(self):
        img = np.zeros((self.h, self.w, 3), np.uint8)
        img[0, 0] = 255                                          # top-left marker: must end up bottom-right
        return {"agentview_image": img, "robot0_eye_in_hand_image": img // 2, "robot0_eef_pos": self.pos.copy(),
                "robot0_eef_quat": np.array([0, 0, np.sin(np.pi / 4), np.cos(np.pi / 4)]),
                "robot0_gripper_qpos": np.array([0.04, -0.04])}

    def reset(self):
        self.pos = self.init.copy() if self.init is not None else np.zeros(3)
        return self._get_observations()

    def step(self, a):
        self.pos = self.pos + 0.1 * np.asarray(a[:3], float)
        return self._get_observations(), 0.0, False, {}

    def check_success(self):
        return self.pos[0] > 0.5

    def close(self):
        pass


class _LiberoBackend:
    def num_tasks(self, suite):
        return 3

    def get_task(self, suite, tid):
        return f"{suite}_task{tid}", f"do thing {tid}", [np.array([0.01 * i, 0, 0]) for i in range(4)]

    def make(self, suite, tid, h, w, freq):
        return _LiberoSim(h, w)


class _Push(torch.nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.p, self.dim = torch.nn.Parameter(torch.zeros(1)), dim

    def reset(self):
        pass

    def select_action(self, batch):
        a = torch.zeros(batch["state"].shape[0], self.dim)
        a[:, 0 if self.dim == 7 else 5] = 1.0
        return a


def test_libero_helpers():
    assert libero.parse_camera_names(" a, b ,") == ["a", "b"] and libero.select_task_ids(4, [3, 1, 1]) == [1, 3]
    with pytest.raises(ValueError):
        libero.select_task_ids(2, [5])
    aa = libero.quat2axisangle([0, 0, np.sin(np.pi / 4), np.cos(np.pi / 4)])
    assert np.allclose(aa, [0, 0, np.pi / 2]) and np.allclose(libero.quat2axisangle([0, 0, 0, 1]), 0)
    s = libero.summarize_libero_results([12, -1, 30, -2])
    assert s["success_rate"] == 0.5 and s["crashed_indices"] == [3] and s["avg_steps_taken_until_success"] == 21.0
    assert libero.get_libero_dummy_action()[-1] == -1


def test_libero_wrapper_and_eval_pipeline():
    cfg = LiberoEnvConfig(task="libero_goal", task_ids=[0, 2], observation_height=32, observation_width=48)
    envs = libero.create_libero_envs(cfg, n_envs=2, backend=_LiberoBackend())
    assert set(envs) == {"libero_goal"} and set(envs["libero_goal"]) == {0, 2}
    venv = envs["libero_goal"][0]
    obs, _ = venv.reset(seed=[1, 2])
    assert obs["pixels"]["camera0"].shape == (2, 32, 48, 3) and obs["agent_pos"].shape == (2, 8)
    assert obs["pixels"]["camera0"][0, -1, -1, 0] == 255 and obs["pixels"]["camera0"][0, 0, 0, 0] == 0   # rotated
    assert np.allclose(obs["agent_pos"][1, :3], [0.01, 0, 0]) and np.allclose(obs["agent_pos"][0, 3:6], [0, 0, np.pi / 2])
    assert venv.call("_max_episode_steps") == (300, 300) and venv.call("task_description")[0] == "do thing 0"
    res = eval_policy(venv, _Push(7), n_episodes=2, start_seed=0, device="cpu")
    assert res["aggregated"]["pc_success"] == 100.0
    with pytest.raises(RuntimeError, match="graphics"):
        make_envs(cfg, 1)                                      # the real simulator is not installed here


class _CasaSim:
    language = "open the drawer"

    def __init__(self):
        self.x = 0.0

    def reset(self):
        return self._obs()

    def _obs(self):
        return {"robot0_agentview_left_image": np.full((16, 16, 3), 7, np.uint8),
                "robot0_eye_in_hand_image": np.full((16, 16, 3), 9, np.uint8),
                "robot0_eef_pos": np.array([self.x, 0, 0]), "robot0_gripper_qpos": np.array([0.1, -0.1])}

    def step(self, a):
        assert set(a) == {"action.base_motion", "action.control_mode", "action.end_effector_position",
                          "action.end_effector_rotation", "action.gripper_close"}
        self.x += 0.2 * float(a["action.end_effector_position"][0])
        return self._obs(), 0.0, False, {}

    def check_success(self):
        return self.x > 0.5

    def close(self):
        pass


class _CasaBackend:
    def make(self, task, split, seed, cameras, h, w):
        return _CasaSim()


def test_robocasa_wrapper_and_eval_pipeline():
    d = robocasa.convert_action(np.arange(12))
    assert d["action.control_mode"].tolist() == [4] and d["action.gripper_close"].tolist() == [11]
    assert robocasa.resolve_tasks("A, B,A") == ["A", "B"] and robocasa.official_task_horizon("CoffeePressButton") == 300
    cfg = RoboCasaEnvConfig(task="OpenDrawer,CloseDrawer", episode_length=20)
    envs = robocasa.create_robocasa_envs(cfg, n_envs=2, backend=_CasaBackend())
    assert list(envs) == ["OpenDrawer", "CloseDrawer"]
    venv = envs["OpenDrawer"][0]
    obs, _ = venv.reset(seed=3)
    assert obs["pixels"]["camera1"][0, 0, 0, 0] == 9 and obs["agent_pos"].shape == (2, 16)
    assert venv.call("task_description")[0] == "open the drawer"
    res = eval_policy(venv, _Push(12), n_episodes=2, start_seed=0, device="cpu")
    assert res["aggregated"]["pc_success"] == 100.0


def test_libero_eval_config_validation():
    from opentau_b200.configs.libero import LiberoEnvConfig, TrainConfigWithLiberoEval
    c = LiberoEnvConfig(suite="libero_goal", id=3)
    assert c.suite == "goal" and c.suite_name == "libero_goal"
    with pytest.raises(ValueError, match="Invalid suite"):
        LiberoEnvConfig(suite="kitchen", id=0)
    with pytest.raises(ValueError, match="Invalid task id"):
        LiberoEnvConfig(suite="object", id=10)
    cfg = TrainConfigWithLiberoEval(libero=LiberoEnvConfig(suite="10", id=2), action_chunk=8)
    assert cfg.libero.chunk_usage == 8
    with pytest.raises(ValueError, match="chunk_usage"):
        TrainConfigWithLiberoEval(libero=LiberoEnvConfig(suite="10", id=2, chunk_usage=9), action_chunk=8)
    with pytest.raises(ValueError, match="must be provided"):
        TrainConfigWithLiberoEval()
