"""Datasets: record -> read round trip (v2.1 images and videos), delta timestamps and padding, standard format,
delta actions, statistics aggregation, VQA samples, <loc> codec, mixture factory and validation split."""

import numpy as np
import pytest
import torch

from opentau_b200.configs.default import DatasetConfig, DatasetMixtureConfig
from opentau_b200.configs.train import TrainPipelineConfig
from opentau_b200.datasets.action_indexing import apply_delta_actions, undo_delta_actions
from opentau_b200.datasets.compute_stats import aggregate_stats, compute_episode_stats
from opentau_b200.datasets.factory import make_dataset, make_dataset_mixture, split_episodes
from opentau_b200.datasets.grounding import loc_tokens_to_xyxy, xyxy_to_loc_tokens
from opentau_b200.datasets.lerobot_dataset import LeRobotDataset, LeRobotDatasetMetadata

FEATURES = {
    "observation.images.top": {"dtype": "image", "shape": (48, 64, 3), "names": ["height", "width", "channel"]},
    "observation.state": {"dtype": "float32", "shape": (6,), "names": None},
    "action": {"dtype": "float32", "shape": (6,), "names": None},
}


def _record(root, use_videos=False, episodes=(12, 9, 15), fps=10):
    rec = LeRobotDataset.create("local/toy", fps=fps, root=root, robot_type="toybot", features=FEATURES,
                                use_videos=use_videos, image_writer_threads=2 if use_videos else 0)
    k = 0
    for e, n in enumerate(episodes):
        for t in range(n):
            img = np.full((48, 64, 3), (k * 3) % 256, dtype=np.uint8)
            rec.add_frame({"observation.images.top": img, "observation.state": np.full(6, k, np.float32),
                           "action": np.full(6, k + 0.5, np.float32), "task": f"task {e % 2}"})
            k += 1
        rec.save_episode()
    rec.stop_image_writer()
    return rec


def _cfg(root, **kw):
    mix = DatasetMixtureConfig(datasets=[DatasetConfig(repo_id="local/toy", root=str(root), **kw.pop("ds", {}))],
                               action_freq=10.0, **kw.pop("mix", {}))
    return TrainPipelineConfig(dataset_mixture=mix, resolution=(56, 56), num_cams=2, action_chunk=5, batch_size=2,
                               dataloader_batch_size=2, **kw)


def test_record_and_read_back(tmp_path):
    _record(tmp_path / "toy")
    meta = LeRobotDatasetMetadata("local/toy", root=tmp_path / "toy")
    assert meta.total_episodes == 3 and meta.total_frames == 36 and meta.fps == 10 and meta.robot_type == "toybot"
    assert meta.tasks == {0: "task 0", 1: "task 1"} and meta.version == "v2.1"
    np.testing.assert_allclose(meta.stats["observation.state"]["mean"], np.full(6, 17.5), rtol=1e-6)
    np.testing.assert_allclose(meta.stats["observation.state"]["max"], np.full(6, 35.0))
    assert meta.stats["observation.images.top"]["mean"].shape == (3, 1, 1)
    cfg = _cfg(tmp_path / "toy")
    ds = make_dataset(cfg.dataset_mixture.datasets[0], cfg)
    assert len(ds) == 36 and ds.num_episodes == 3
    s = ds[10]                                   # episode 0, frame 10 of 12: two chunk steps run past the end
    assert s["camera0"].shape == (3, 56, 56) and s["camera0"].dtype == torch.bfloat16
    assert s["img_is_pad"].tolist() == [False, True] and float(s["camera1"].abs().sum()) == 0.0
    assert s["state"].shape == (32,) and float(s["state"][0]) == 10.0 and float(s["state"][6]) == 0.0
    assert s["actions"].shape == (5, 32) and s["actions"][:, 0].float().tolist() == [10.5, 11.5, 11.5, 11.5, 11.5]
    assert s["action_is_pad"].tolist() == [False, False, True, True, True]
    assert int(s["real_action_dim"]) == 6 and s["prompt"] == "task 0" and s["response"] == ""
    assert s["episode_index"] == 0 and s["frame_index"] == 10 and s["source"] == "local/toy"
    # the picture is letter-boxed: 64x48 -> 56x42 centred, rows outside are the pad value
    assert float(s["camera0"][0, 0, 0]) == 0.0 and abs(float(s["camera0"][0, 28, 28]) - 30 / 255) < 1e-2
    assert ds[12]["prompt"] == "task 1" and ds[12]["frame_index"] == 0


def test_video_backed_dataset_and_history(tmp_path):
    _record(tmp_path / "toy", use_videos=True)
    assert (tmp_path / "toy" / "videos/chunk-000/observation.images.top/episode_000001.mp4").exists()
    cfg = _cfg(tmp_path / "toy", mix=dict(n_obs_history=3))
    ds = make_dataset(cfg.dataset_mixture.datasets[0], cfg)
    s = ds[13]                                   # episode 1, frame 1: one of three history frames is before the start
    assert s["camera0"].shape == (3, 3, 56, 56) and s["state"].shape == (3, 32)
    assert s["obs_history_is_pad"].tolist() == [True, False, False]
    assert s["state"][:, 0].float().tolist() == [12.0, 12.0, 13.0]
    centre = s["camera0"][:, 0, 28, 28].float() * 255
    assert torch.allclose(centre, torch.tensor([36.0, 36.0, 39.0]), atol=6.0)   # lossy codec


def test_column_index_and_delta_actions(tmp_path):
    _record(tmp_path / "toy")
    cfg = _cfg(tmp_path / "toy", ds=dict(state_index=[0, 1], action_index=[2, 3, 4], use_delta_joint_actions=True,
                                         delta_action_state_map={"0": 1}))
    s = make_dataset(cfg.dataset_mixture.datasets[0], cfg)[3]
    assert int(s["real_action_dim"]) == 3
    assert s["actions"][:3, :3].float().tolist() == [[0.5, 3.5, 3.5], [1.5, 4.5, 4.5], [2.5, 5.5, 5.5]]
    a, st = torch.randn(2, 5, 4), torch.randn(2, 3)
    d = torch.stack([apply_delta_actions(a[i], st[i], {1: 2}) for i in range(2)])
    assert torch.allclose(undo_delta_actions(d, st, {1: 2}), a, atol=1e-6)


def test_stats_aggregation_matches_pooled_data():
    rng = np.random.default_rng(0)
    feats = {"x": {"dtype": "float32", "shape": (3,)}}
    parts = [rng.normal(i, 1 + i, size=(n, 3)) for i, n in enumerate((10, 40, 7))]
    agg = aggregate_stats([compute_episode_stats({"x": p}, feats) for p in parts])["x"]
    pooled = np.concatenate(parts)
    np.testing.assert_allclose(agg["mean"], pooled.mean(0), rtol=1e-10)
    np.testing.assert_allclose(agg["std"], pooled.std(0), rtol=1e-10)
    np.testing.assert_allclose(agg["min"], pooled.min(0))
    assert int(agg["count"][0]) == 57


def test_split_is_deterministic_and_disjoint():
    eps = list(range(20))
    a, b = split_episodes(eps, 0.2, 7, "x/y"), split_episodes(eps, 0.2, 7, "x/y")
    assert a == b and len(a[1]) == 4 and not set(a[0]) & set(a[1]) and sorted(a[0] + a[1]) == eps
    assert split_episodes(eps, 0.2, 8, "x/y") != a


def test_loc_codec_round_trip():
    s = xyxy_to_loc_tokens([(10, 20, 110, 220)], ["cup"], (640, 480))
    assert s == "<loc0043><loc0016><loc0469><loc0176> cup"
    (box, label), = loc_tokens_to_xyxy(s, (640, 480))
    assert label == "cup" and np.allclose(box, (10, 20, 110, 220), atol=0.5)


def test_mixture_with_vqa_and_validation_split(tmp_path):
    _record(tmp_path / "toy", episodes=(8, 8, 8, 8))
    mix = DatasetMixtureConfig(datasets=[DatasetConfig(repo_id="local/toy", root=str(tmp_path / "toy")),
                                         DatasetConfig(vqa="dummy")], weights=[0.7, 0.3], action_freq=10.0,
                               val_split_ratio=0.25)
    cfg = TrainPipelineConfig(dataset_mixture=mix, resolution=(56, 56), num_cams=1, action_chunk=5, batch_size=4,
                              dataloader_batch_size=4, val_freq=10, num_workers=0)
    train, val = make_dataset_mixture(cfg)
    assert len(train.meta.per_dataset_stats) == 2 and train.meta.dataset_to_norm_index == {"local/toy": 0, "dummy": 1}
    batch = next(iter(train.get_dataloader(4, num_workers=0)))
    assert batch["camera0"].shape == (4, 3, 56, 56) and batch["actions"].shape == (4, 5, 32)
    assert set(batch["dataset_index"].tolist()) <= {0, 1} and len(batch["prompt"]) == 4
    vq = [i for i, n in enumerate(batch["dataset_repo_id"]) if n == "dummy"]
    assert all(bool(batch["action_is_pad"][i].all()) for i in vq)
    assert len(val) > 0 and val.datasets[0].dataset.train is False


def test_missing_dataset_raises_clear_error(tmp_path):
    with pytest.raises(FileNotFoundError, match="no network"):
        LeRobotDatasetMetadata("nobody/nothing", root=tmp_path / "absent")


def test_push_to_hub_helpers(tmp_path):
    import pytest

    from opentau_b200.datasets.push_dataset_to_hub.utils import (calculate_episode_data_index, check_repo_id,
                                                                  concatenate_episodes, get_default_encoding,
                                                                  save_images_concurrently)
    eps = [{"frame_index": torch.arange(3), "action": torch.ones(3, 2), "task": ["a"] * 3},
           {"frame_index": torch.arange(2), "action": torch.zeros(2, 2), "task": ["b"] * 2}]
    cat = concatenate_episodes(eps)
    assert cat["index"].tolist() == [0, 1, 2, 3, 4] and cat["action"].shape == (5, 2) and cat["task"][3] == "b"
    idx = calculate_episode_data_index([0, 0, 0, 1, 1, 1, 1, 2, 2, 2, 2, 2])
    assert idx["from"].tolist() == [0, 3, 7] and idx["to"].tolist() == [3, 7, 12]
    assert calculate_episode_data_index({"episode_index": []})["from"].numel() == 0
    paths = save_images_concurrently(np.zeros((3, 4, 5, 3), np.uint8), tmp_path / "imgs", max_workers=2)
    assert [p.name for p in paths] == ["frame_000000.png", "frame_000001.png", "frame_000002.png"]
    assert all(p.exists() for p in paths)
    check_repo_id("lerobot/pusht")
    for bad in ("pusht", "a/b/c", "/x"):
        with pytest.raises(ValueError):
            check_repo_id(bad)
    assert isinstance(get_default_encoding(), dict)
