"""Evaluation pipeline on the headless environment: a scripted policy that drives towards the goal succeeds, a
policy that stands still does not; per-task / per-group aggregation; the trained-policy path with a tiny pi0.5."""

import numpy as np
import torch

from helpers import tiny_pi05
from opentau_b200.envs import FakeEnvConfig, make_envs, preprocess_observation
from opentau_b200.scripts.eval import consolidate_eval_info, eval_policy, eval_policy_all, rollout
from opentau_b200.scripts.launch import build_command


class Scripted(torch.nn.Module):
    def __init__(self, gain):
        super().__init__()
        self.p = torch.nn.Parameter(torch.zeros(1))
        self.gain = gain

    def reset(self):
        pass

    def select_action(self, batch):
        st = batch["state"]
        return self.gain * (st[:, 4:8] - st[:, 0:4]) * 4.0


def test_rollout_shapes_and_success_accounting():
    cfg = FakeEnvConfig(tasks=["reach a", "reach b"], task_groups={"easy": [0], "hard": [1]}, episode_length=30)
    envs = make_envs(cfg, n_envs=3)
    env = envs["easy"][0]
    data = rollout(env, Scripted(1.0), seeds=[1, 2, 3], device="cpu")
    assert data["action"].shape[0] == 3 and data["action"].shape[2] == 4 and data["done"][:, -1].all()
    good = eval_policy(env, Scripted(1.0), n_episodes=5, start_seed=10, device="cpu")
    bad = eval_policy(env, Scripted(0.0), n_episodes=5, start_seed=10, device="cpu")
    assert good["aggregated"]["pc_success"] == 100.0 and bad["aggregated"]["pc_success"] == 0.0
    assert len(good["per_episode"]) == 5 and good["per_episode"][4]["seed"] == 14
    assert good["aggregated"]["avg_sum_reward"] > bad["aggregated"]["avg_sum_reward"]
    r0 = eval_policy_all(envs, Scripted(1.0), 3, 0, device="cpu", rank=0, world=2)
    r1 = eval_policy_all(envs, Scripted(0.0), 3, 0, device="cpu", rank=1, world=2)
    assert set(r0) == {"easy/0"} and set(r1) == {"hard/1"}
    info = consolidate_eval_info([r0, r1])
    assert info["per_group"]["easy"]["pc_success"] == 100.0 and info["per_group"]["hard"]["pc_success"] == 0.0
    assert info["aggregated"]["pc_success"] == 50.0 and info["aggregated"]["n"] == 6


def test_observation_preprocessing_and_real_policy():
    cfg = FakeEnvConfig(state_dim=8, action_dim=4, resolution=(224, 224), episode_length=3)
    env = make_envs(cfg, n_envs=2)["reach"][0]
    obs, _ = env.reset(seed=0)
    b = preprocess_observation(obs)
    assert b["camera0"].shape == (2, 3, 224, 224) and b["camera0"].max() <= 1.0 and b["state"].shape == (2, 8)
    pol = tiny_pi05().eval()

    class Pad:                       # env states are 8 wide, the policy expects max_state_dim
        max_state_dim = 32
    res = eval_policy(env, pol, n_episodes=2, start_seed=0, cfg=Pad, device="cpu")
    assert len(res["per_episode"]) == 2 and np.isfinite(res["aggregated"]["avg_sum_reward"])


def test_launcher_commands():
    cmd, env = build_command("opentau_b200.scripts.train", ["--num-processes", "4", "--steps=3"])
    assert cmd[1:4] == ["-m", "torch.distributed.run", "--nnodes=1"] and "--nproc-per-node=4" in cmd
    assert cmd[-3:] == ["-m", "opentau_b200.scripts.train", "--steps=3"] and "127.0.0.1" in cmd
    cmd, _ = build_command("opentau_b200.scripts.eval", ["--num_processes=1", "--x=1"])
    assert cmd[1:] == ["-m", "opentau_b200.scripts.eval", "--x=1"]


def test_subgoal_generators_feed_the_rollout(tmp_path):
    """The dataset-backed generator serves the last frame of an episode with the environment's task string; the
    goal-frame generator indexes pre-rendered frames by the rollout seed; both reach the policy at every step."""
    from PIL import Image
    from opentau_b200.envs.subgoal import GoalFrameSubgoalGenerator, LastFrameSubgoalGenerator
    from test_datasets_cpu import _record
    import pytest
    _record(tmp_path / "toy", episodes=(5, 7, 4))                 # tasks: "task 0", "task 1", "task 0"
    gen = LastFrameSubgoalGenerator(tmp_path / "toy", resolution=(32, 32), seed=0)
    assert gen.known_languages == ["task 0", "task 1"]
    envs = make_envs(FakeEnvConfig(tasks=["task 1"], episode_length=6), n_envs=2)
    env = envs[next(iter(envs))][0]
    seen = []

    class Watch(Scripted):
        def select_action(self, batch):
            seen.append((batch["subgoal0"].clone(), batch["subgoal_is_pad"].clone()))
            return super().select_action(batch)

    rollout(env, Watch(1.0), seeds=[3, 4], device="cpu", subgoal_generator=gen)
    sg, pad = seen[0]
    assert sg.shape == (2, 3, 32, 32) and not pad.any() and len(seen) >= 1
    # episode 1 (the only "task 1" episode) ends at global frame 11 -> pixel value (11 * 3) % 256 = 33
    assert abs(float(sg[0, 0, 20, 16]) * 255 - 33) < 1.5 and torch.equal(seen[0][0], seen[-1][0])
    with pytest.raises(ValueError, match="no episode"):
        gen.start_episode(["unknown task"])
    for s in range(3):
        (tmp_path / "goals" / f"scene_{s}").mkdir(parents=True)
        Image.fromarray(np.full((32, 32, 3), 50 * s, np.uint8)).save(tmp_path / "goals" / f"scene_{s}" / "0.png")
    goals = GoalFrameSubgoalGenerator(tmp_path / "goals", resolution=(32, 32))
    goals.start_episode(["a", "b"], seeds=[4, 2])
    out = goals({"state": torch.zeros(2, 8)})
    assert goals.num_scenes == 3 and abs(float(out["subgoal0"][0, 0, 0, 0]) * 255 - 50) < 1 \
        and abs(float(out["subgoal0"][1, 0, 0, 0]) * 255 - 100) < 1


def test_rollouts_become_a_dataset(tmp_path):
    """Two rollouts (one succeeding, one standing still) are merged and written as episodes cut at the first done,
    with the outcome in the episode metadata; the result loads like any recorded dataset."""
    from opentau_b200.datasets.lerobot_dataset import LeRobotDatasetMetadata
    from opentau_b200.utils.rollout_recorder import aggregate_rollouts, record_rollouts
    envs = make_envs(FakeEnvConfig(tasks=["reach the goal"], episode_length=12), n_envs=2)
    env = envs[next(iter(envs))][0]
    good = rollout(env, Scripted(1.0), seeds=[1, 2], device="cpu", return_observations=True)
    bad = rollout(env, Scripted(0.0), seeds=[3, 4], device="cpu", return_observations=True)
    data = aggregate_rollouts([good, bad])
    assert data["done"].shape[0] == 4 and len(data["observation"]) == data["done"].shape[1]
    rep = record_rollouts(data, tmp_path / "ds", fps=10, prompts=["reach the goal"] * 4)
    assert rep["episodes"] == 4 and rep["successes"] == 2
    meta = LeRobotDatasetMetadata("ds", root=tmp_path / "ds")
    assert meta.total_episodes == 4 and meta.total_frames == rep["frames"] and meta.tasks[0] == "reach the goal"
    assert [meta.episodes[i]["success"] for i in range(4)] == [True, True, False, False]
    assert meta.episodes[2]["length"] == 12 and meta.episodes[0]["length"] < 12          # success ends the episode early
    only = record_rollouts(data, tmp_path / "ok", fps=10, prompts=["reach the goal"] * 4, only_successful=True)
    assert only["episodes"] == 2 and only["successes"] == 2
