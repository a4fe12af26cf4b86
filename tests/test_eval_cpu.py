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


def test_videos_grid_summary_goal_frames_and_accel_streams(tmp_path):
    """Everything the evaluator builds from frame arrays: per-episode clips tiled into a grid video whose held last
    frame carries a green / red border per tile, the final camera frames of successful episodes keyed by seed, and
    the accel values a policy publishes per chunk."""
    import cv2
    from opentau_b200.scripts.eval import create_grid_summary_video, write_video
    cfg = FakeEnvConfig(tasks=["reach"], episode_length=12, resolution=(64, 64))
    env = make_envs(cfg, n_envs=2)["reach"][0]

    class WithAccel(Scripted):
        def __init__(self, gain):
            super().__init__(gain)
            self.last_accel, self.last_accel_provenance, self.n = None, {"prefix": 5}, 0

        def select_action(self, batch):
            self.n += 1
            if self.n % 3 == 1:                                   # a new chunk every third step
                self.last_accel = torch.full((2,), float(self.n))
            return super().select_action(batch)

    res = eval_policy(env, WithAccel(1.0), n_episodes=3, start_seed=5, device="cpu", max_episodes_rendered=3,
                      videos_dir=tmp_path / "videos", goal_frames_dir=tmp_path / "goals", task_name="reach_0")
    assert res["aggregated"]["pc_success"] == 100.0
    grid = tmp_path / "videos" / "grid_summary.mp4"
    assert grid.exists() and res["video_paths"] == [str(grid)] and not list((tmp_path / "videos").glob("eval_episode_*"))
    cap = cv2.VideoCapture(str(grid))
    n, last = 0, None
    while True:
        ok, f = cap.read()
        if not ok:
            break
        n, last = n + 1, f
    assert n > 10 and last.shape[:2] == (128, 128)                # 3 clips -> 2 x 2 tiles of 64 x 64
    assert last[2, 30, 1] > 120 and last[2, 30, 2] < 90           # green border on a successful tile (BGR)
    assert len(res["goal_frames"]) == 3 and {r["seed"] for r in res["goal_frames"]} == {5, 6, 7}
    png = cv2.imread(str(tmp_path / "goals" / res["goal_frames"][0]["camera0"]))
    assert png is not None and png.shape[:2] == (64, 64)
    assert (tmp_path / "goals" / "manifest_rank0.jsonl").read_text().count("\n") == 3
    streams = res["accel"]["streams"]
    assert len(streams) == 3 and all(len(s) >= 1 for s in streams) and res["accel"]["provenance"] == {"prefix": 5}
    # a failed tile gets a red border; a clip that ends early keeps its last frame
    a, b = tmp_path / "a.mp4", tmp_path / "b.mp4"
    write_video(a, np.full((4, 32, 32, 3), 200, np.uint8), 10)
    write_video(b, np.full((9, 32, 32, 3), 50, np.uint8), 10)
    create_grid_summary_video([str(a), str(b)], [False, True], tmp_path / "g.mp4", 10, highlight_duration=0.5,
                              grid_size=(1, 2), frame_stride=2)
    cap = cv2.VideoCapture(str(tmp_path / "g.mp4"))
    frames = []
    while True:
        ok, f = cap.read()
        if not ok:
            break
        frames.append(f)
    assert len(frames) == 5 + 5 and frames[-1][1, 10, 2] > 150 and frames[-1][1, 10, 1] < 90     # red on tile 0
    assert frames[3][16, 16].mean() > 150                         # tile 0 still shows its last frame after it ended


def test_seed_blocks_resolution_check_and_grid_collection(tmp_path):
    import pytest

    from helpers import tiny_pi05_config
    from opentau_b200.configs.train import TrainPipelineConfig
    from opentau_b200.scripts.eval import _rank_seed_offset, collect_grid_summary_videos, validate_eval_input_resolution
    # off: every rank seeds alike; on: blocks of exactly one rank's span tile the seed line
    assert [_rank_seed_offset(r, False, 40) for r in range(3)] == [0, 0, 0]
    blocks = [range(_rank_seed_offset(r, True, 40), _rank_seed_offset(r, True, 40) + 40) for r in range(4)]
    assert all(blocks[i].stop == blocks[i + 1].start for i in range(3))
    # frames reach the tower at cfg.resolution: only a policy WITHOUT a resize target can be silently wrong
    pol = tiny_pi05_config(resize_imgs_with_padding=None)
    cfg = TrainPipelineConfig(policy=pol, resolution=(224, 224))
    validate_eval_input_resolution(cfg)
    cfg.resolution = (128, 128)
    with pytest.raises(ValueError, match="wrong geometry"):
        validate_eval_input_resolution(cfg)
    pol.skip_input_resolution_check = True
    validate_eval_input_resolution(cfg)
    cfg.policy = tiny_pi05_config(resize_imgs_with_padding=(224, 224))
    validate_eval_input_resolution(cfg)                               # a resize target corrects the frames
    assert cfg.policy.input_image_size == (224, 224)
    for name in ("libero_3_rank0", "libero_1_rank12", "robocasa_7"):
        (tmp_path / name).mkdir()
        (tmp_path / name / "grid_summary.mp4").write_bytes(b"x")
        (tmp_path / name / "eval_episode_0.mp4").write_bytes(b"x")
    got = collect_grid_summary_videos(tmp_path)
    assert [g[0] for g in got] == ["libero_1", "libero_3", "robocasa_7"] and all(g[1].endswith("grid_summary.mp4") for g in got)
    assert collect_grid_summary_videos(tmp_path / "absent") == []


def test_environment_metadata_reaches_the_batch():
    import pytest
    import torch

    from opentau_b200.envs.configs import EnvMetadataConfig, FakeEnvConfig
    from opentau_b200.envs.utils import add_eval_metadata, close_envs
    from opentau_b200.scripts.eval import resolve_env_config
    env = resolve_env_config({"type": "fake", "fps": 20, "metadata": {"speed": 30, "mistake": False, "control_mode": "ee",
                                                                      "emit_fps": True}})
    assert isinstance(env, FakeEnvConfig) and env.metadata.speed == 30
    obs = add_eval_metadata({"state": torch.zeros(3, 8)}, env)
    assert obs["speed"].tolist() == [30] * 3 and obs["speed"].dtype == torch.long and not obs["speed_is_pad"].any()
    assert obs["mistake"].tolist() == [False] * 3 and obs["mistake"].dtype == torch.bool        # False is a value
    assert obs["control_mode"] == ["ee"] * 3 and "quality" not in obs and "robot_type" not in obs
    assert obs["fps"].tolist() == [20] * 3 and not obs["fps_is_pad"].any()
    assert set(add_eval_metadata({"state": torch.zeros(2, 8)}, FakeEnvConfig())) == {"state"}     # all None: nothing added
    for bad, err in ((dict(speed=35), ValueError), (dict(speed=True), TypeError), (dict(quality=0), ValueError),
                     (dict(quality=2.0), TypeError), (dict(mistake=1), TypeError), (dict(robot_type=""), ValueError),
                     (dict(control_mode="torque"), ValueError)):
        with pytest.raises(err):
            EnvMetadataConfig(**bad)

    class E:
        def __init__(self, fail=False):
            self.closed, self.fail = False, fail

        def close(self):
            self.closed = True
            if self.fail:
                raise RuntimeError("boom")
    envs = {"suite": {0: E(), 1: E(fail=True)}, "other": [E(), None]}
    close_envs(envs)                                                   # one failure does not keep the others open
    assert all(e.closed for e in (*envs["suite"].values(), envs["other"][0]))
