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
    kw.setdefault("num_cams", 2)
    return TrainPipelineConfig(dataset_mixture=mix, resolution=(56, 56), action_chunk=5, batch_size=2,
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
                                         delta_action_state_map={"2": 1}))   # stored action column 2 (emitted 0), state column 1
    ds = make_dataset(cfg.dataset_mixture.datasets[0], cfg)
    s = ds[3]
    assert int(s["real_action_dim"]) == 3
    assert s["actions"][:3, :3].float().tolist() == [[0.5, 3.5, 3.5], [1.5, 4.5, 4.5], [2.5, 5.5, 5.5]]
    # the statistics that normalise these targets describe the DELTAS (computed from the columns, cached beside the
    # dataset) and reach the mixture's head in the emitted layout, padded
    assert ds.delta_action_state_map == {0: 1}
    every = torch.stack([ds[i]["actions"][:, :3].float() for i in range(len(ds))])
    got = ds.delta_action_stats["actions"]
    assert np.allclose(got["mean"], every.reshape(-1, 3).mean(0).numpy(), atol=1e-4)
    assert np.allclose(got["min"], every.reshape(-1, 3).amin(0).numpy(), atol=1e-5)
    assert len(list((tmp_path / "toy" / "meta" / "delta_action_stats").glob("*.json"))) == 1
    mix = make_dataset_mixture(cfg)
    head = mix.meta.per_norm_key_stats[0]["actions"]
    assert head["mean"].shape == (32,) and np.allclose(head["mean"][:3], got["mean"]) and np.all(head["mean"][3:] == 0)
    assert mix.meta.delta_action_state_map == {0: 1} and mix.meta.per_norm_key_stats[0]["state"]["mean"].shape == (32,)
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
    with pytest.raises(FileNotFoundError, match="could not be fetched"):
        LeRobotDatasetMetadata("nobody/nothing", root=tmp_path / "absent")
    assert not (tmp_path / "absent").exists()


class _FakeHub:
    """Serves files out of a source folder and records every call."""

    def __init__(self, source):
        self.source, self.calls = source, []

    def snapshot_download(self, repo_id, *, revision, local_dir, allow_patterns=None, ignore_patterns=None):
        import shutil
        self.calls.append(("snapshot", allow_patterns, ignore_patterns))
        for f in self.source.rglob("*"):
            rel = f.relative_to(self.source).as_posix()
            if not f.is_file() or (allow_patterns and not rel.startswith(allow_patterns)) \
                    or (ignore_patterns and rel.startswith(ignore_patterns)):
                continue
            (local_dir / rel).parent.mkdir(parents=True, exist_ok=True)
            shutil.copy(f, local_dir / rel)

    def download_file(self, repo_id, filename, *, revision, local_dir):
        import shutil
        self.calls.append(("file", filename))
        (local_dir / filename).parent.mkdir(parents=True, exist_ok=True)
        shutil.copy(self.source / filename, local_dir / filename)

    def create_repo(self, repo_id, *, private):
        self.calls.append(("create_repo", repo_id, private))

    def create_branch(self, repo_id, branch, *, revision):
        self.calls.append(("create_branch", branch))

    def upload_folder(self, repo_id, folder, *, revision, allow_patterns=None, ignore_patterns=None, large=False):
        self.calls.append(("upload_folder", str(folder), revision, tuple(ignore_patterns), large))

    def file_exists(self, repo_id, filename, *, revision):
        return False

    def upload_text(self, repo_id, filename, text, *, revision):
        self.calls.append(("upload_text", filename, text))

    def retag(self, repo_id, tag, *, revision):
        self.calls.append(("retag", tag, revision))


def test_hub_transfer_fetches_only_what_is_missing(tmp_path):
    from opentau_b200.datasets.hub_transfer import set_hub_client
    _record(tmp_path / "origin", use_videos=True)
    hub = _FakeHub(tmp_path / "origin")
    set_hub_client(hub)
    try:
        # nothing on disk: the metadata folder comes first, then exactly the selected episodes' files
        meta = LeRobotDatasetMetadata("local/toy", root=tmp_path / "copy")
        assert hub.calls == [("snapshot", "meta/", None)] and meta.total_episodes == 3
        cfg = _cfg(tmp_path / "copy")
        ds = LeRobotDataset(cfg, "local/toy", root=tmp_path / "copy", episodes=[1])
        fetched = sorted(c[1] for c in hub.calls if c[0] == "file")
        assert fetched == ["data/chunk-000/episode_000001.parquet", "videos/chunk-000/observation.images.top/episode_000001.mp4"]
        assert len(ds) == 9
        hub.calls.clear()
        LeRobotDataset(cfg, "local/toy", root=tmp_path / "copy", episodes=[1])           # complete: no request at all
        assert hub.calls == []
        LeRobotDataset(cfg, "local/toy", root=tmp_path / "copy")                         # all episodes: one snapshot
        assert hub.calls == [("snapshot", None, None)]
        hub.calls.clear()
        ds.push_to_hub(branch="v2", tags=["toy"], push_videos=False, private=True)
        kinds = [c[0] for c in hub.calls]
        assert kinds == ["create_repo", "create_branch", "upload_folder", "upload_text", "retag"]
        assert hub.calls[2][3] == ("images/", "videos/") and hub.calls[2][2] == "v2"
        card = hub.calls[3][2]
        assert card.startswith("---") and "- toy" in card and "| total_episodes | 3 |" in card and "| robot_type | toybot |" in card
    finally:
        set_hub_client(None)


def test_hub_revision_resolution(tmp_path, caplog):
    """Which ref is downloaded for a wanted version (reference ``src/opentau/datasets/utils.py:1004-1110``)."""
    from opentau_b200.datasets import hub_transfer as H
    from opentau_b200.datasets.utils import BackwardCompatibilityError

    class Refs(_FakeHub):
        def __init__(self, source, branches, tags):
            super().__init__(source)
            self.branches, self.tags, self.revisions = branches, tags, []

        def list_refs(self, repo_id):
            return list(self.branches), list(self.tags)

        def snapshot_download(self, repo_id, *, revision, **kw):
            self.revisions.append(revision)
            return super().snapshot_download(repo_id, revision=revision, **kw)

    def resolve(branches, tags, want="v2.1", **kw):
        H.set_hub_client(Refs(tmp_path, branches, tags))
        return H.get_safe_version("a/b", want, **kw)

    try:
        assert resolve(["main"], ["v2.0", "v2.1", "v3.0"]) == "v2.1"                 # carried as asked
        with caplog.at_level("WARNING"):
            assert resolve(["main"], ["v2.0", "v1.6"]) == "v2.0"                     # same major, older minor
        assert "not found, using v2.0" in caplog.text
        assert resolve(["main"], ["v3.0"]) == "v3.0"                                 # newer but still readable
        assert resolve(["main", "v2.1"], []) == "v2.1"                               # a version BRANCH counts
        with pytest.raises(H.ForwardCompatibilityError, match="v4.0"):
            resolve(["main"], ["v4.0"])
        with pytest.raises(BackwardCompatibilityError, match="v1.6"):
            resolve(["main"], ["v1.6"])
        with pytest.raises(H.RevisionNotFoundError, match="tagged"):
            resolve(["main"], [])
        assert resolve(["master", "dev"], [], allow_branch_fallback=True) == "master"
        with pytest.raises(H.RevisionNotFoundError):
            resolve(["dev"], [], allow_branch_fallback=True)
        assert H.get_repo_versions("a/b") == []
        # through the dataset: an unpinned revision resolves once, a pinned branch name is used as it is
        _record(tmp_path / "origin", use_videos=False)
        hub = Refs(tmp_path / "origin", ["main"], ["v2.0", "v2.1"])
        H.set_hub_client(hub)
        LeRobotDatasetMetadata("local/toy", root=tmp_path / "copy")
        LeRobotDatasetMetadata("local/toy", root=tmp_path / "copy2", revision="experiment")
        assert hub.revisions == ["v2.1", "experiment"]
    finally:
        H.set_hub_client(None)


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


def test_selection_segments_memory_subgoals_and_optional_keys(tmp_path):
    """Deny list and selected-episode statistics; segment tables from start frames; the memory of the next frame; subgoal
    frame choice (end of segment, 4 s window, legacy look-ahead); every optional key always present with the documented
    pad signals; history dropout; the validation copy shares data and differs only in its switches."""
    from opentau_b200.datasets.lerobot_dataset import aggregate_selected_stats, resolve_selected_episodes
    from opentau_b200.datasets.utils import EPISODES_PATH, load_jsonlines, write_jsonlines
    _record(tmp_path / "toy", episodes=(12, 9, 15))
    eps = load_jsonlines(tmp_path / "toy" / EPISODES_PATH)
    eps[0]["segments"] = [0, 5, 9]
    write_jsonlines(eps, tmp_path / "toy" / EPISODES_PATH)

    assert resolve_selected_episodes(range(3), None, None) is None
    assert resolve_selected_episodes(range(3), [2, 0], None) == [0, 2]
    assert resolve_selected_episodes(range(3), [0, 1], [1]) == [0]                # the deny list wins
    assert resolve_selected_episodes(range(3), None, [1]) == [0, 2]
    with pytest.raises(ValueError, match="removed every episode"):
        resolve_selected_episodes(range(3), [1], [1], "local/toy")
    meta = LeRobotDatasetMetadata("local/toy", root=tmp_path / "toy")
    full = meta.stats["observation.state"]["mean"].copy()
    sel = aggregate_selected_stats(meta, None, [1])["observation.state"]["mean"]
    np.testing.assert_allclose(sel, np.full(6, (np.arange(12).sum() + np.arange(21, 36).sum()) / 27.0), rtol=1e-6)
    assert not np.allclose(sel, full) and aggregate_selected_stats(meta) is meta.stats

    mixkw = dict(subgoal_drop_prob=0.0, subgoal_end_of_segment_prob=1.0, response_drop_prob=0.0,
                 metadata_drop_all_prob=0.0, metadata_drop_each_prob=0.0, history_state_drop_prob=0.0, emit_fps=True)
    cfg = _cfg(tmp_path / "toy", mix=mixkw, ds=dict(excluded_episodes=[1]))
    ds = make_dataset(cfg.dataset_mixture.datasets[0], cfg)
    assert ds.episodes == [0, 2] and len(ds) == 27
    np.testing.assert_allclose(ds.meta.stats["observation.state"]["mean"], sel, rtol=1e-6)   # what the normaliser pools
    assert ds.segment_starts_by_episode[0].tolist() == [0, 5, 9] and ds.segment_starts_by_episode[2].tolist() == [0]
    assert [ds._lookup_segment_index(0, f) for f in (0, 4, 5, 8, 9, 11)] == [0, 0, 1, 1, 2, 2]
    assert ds._segment_end_in_ep(0, 0) == 5 and ds._segment_end_in_ep(0, 2) == 12
    assert ds._sample_subgoal_frame(0, 2, at_end_of_segment=True) == 4
    assert all(6 <= ds._sample_subgoal_frame(0, 6, at_end_of_segment=False) <= 8 for _ in range(20))
    assert ds._sample_subgoal_frame(2, 3, at_end_of_segment=True) == 14         # no annotation: 4 s ahead, clipped
    ds.segment_memories_by_episode[0] = ["m0", "m1", "m2"]
    assert ds._lookup_next_memory(0, 3) == "m0" and ds._lookup_next_memory(0, 4) == "m1"
    assert ds._lookup_next_memory(0, 11) == "m2"
    assert set(ds.speed_raw_by_episode.values()) == {50}                         # two tasks, too few episodes to rank
    assert (tmp_path / "toy" / "meta" / "speed_percentiles.jsonl").exists()

    s = ds[2]
    for k in ("subgoal0", "subgoal1", "subgoal_is_pad", "memory", "next_memory", "speed", "speed_is_pad", "mistake",
              "mistake_is_pad", "quality", "quality_is_pad", "robot_type", "control_mode", "fps", "fps_is_pad",
              "obs_history_is_pad"):
        assert k in s, k
    # one camera of two is mapped, so the subgoals are padded as a whole (all-or-none) and zero-filled
    assert bool(s["subgoal_is_pad"]) and float(s["subgoal0"].float().abs().sum()) == 0.0
    assert int(s["speed"]) == 50 and not bool(s["speed_is_pad"]) and bool(s["quality_is_pad"]) and int(s["quality"]) == 0
    assert s["robot_type"] == "toybot" and s["memory"] == "" and int(s["fps"]) == 10 and not bool(s["fps_is_pad"])

    cfg1 = _cfg(tmp_path / "toy", mix=mixkw, num_cams=1)
    ds1 = make_dataset(cfg1.dataset_mixture.datasets[0], cfg1)
    s1 = ds1[2]
    assert not bool(s1["subgoal_is_pad"]) and s1["subgoal0"].shape == (3, 56, 56)
    assert abs(float(s1["subgoal0"].float()[0, 28, 28]) * 255 - 12) < 2          # frame 4 = last frame of segment 0
    val = ds1.shallow_copy_with_dropout(enable_dropout=False, enable_prompt_substitution=False)
    assert val._table is ds1._table and val.meta is ds1.meta and not val.enable_optional_key_dropout
    assert ds1.enable_optional_key_dropout and ds1.enable_prompt_substitution
    ds1.cfg.dataset_mixture.history_state_drop_prob = 1.0
    assert bool(ds1[2]["obs_history_is_pad"].all()) and not bool(val[2]["obs_history_is_pad"].any())
    ds1.cfg.dataset_mixture.subgoal_drop_prob = 1.0
    assert bool(ds1[2]["subgoal_is_pad"]) and not bool(val[2]["subgoal_is_pad"])
    with pytest.raises(AssertionError, match=r"\(3, H, W\)"):
        ds1._assert_image_in_unit_range(torch.full((3, 4, 4), 1.5), name="x", expect_temporal=False)


def test_deferred_videos_are_attached_after_recording(tmp_path):
    """A video feature declared as deferred takes no frames in ``add_frame``; a clip recorded elsewhere is re-timed to
    the dataset's rate, cut to the episode's length and placed at the standard path; the metadata then gets the real
    video properties and the dataset reads the frames back."""
    import cv2
    feats = {**FEATURES, "observation.images.wrist": {"dtype": "video", "shape": (48, 64, 3), "names": ["h", "w", "c"]}}
    rec = LeRobotDataset.create("local/toy", fps=10, root=tmp_path / "toy", robot_type="toybot", features=feats,
                                use_videos=True, image_writer_threads=2, deferred_video_keys={"observation.images.wrist"})
    with pytest.raises(ValueError, match="not video features"):
        LeRobotDataset.create("local/x", fps=10, root=tmp_path / "x", features=feats, use_videos=True,
                              deferred_video_keys={"nope"})
    for t in range(8):
        rec.add_frame({"observation.images.top": np.full((48, 64, 3), 10 * t, np.uint8),
                       "observation.state": np.full(6, t, np.float32), "action": np.full(6, t, np.float32), "task": "go"})
    with pytest.raises(ValueError, match="deferred video keys"):
        rec.add_frame({"observation.images.top": np.zeros((48, 64, 3), np.uint8),
                       "observation.images.wrist": np.zeros((48, 64, 3), np.uint8),
                       "observation.state": np.zeros(6, np.float32), "action": np.zeros(6, np.float32), "task": "go"})
    rec.clear_episode_buffer()
    for t in range(8):
        rec.add_frame({"observation.images.top": np.full((48, 64, 3), 10 * t, np.uint8),
                       "observation.state": np.full(6, t, np.float32), "action": np.full(6, t, np.float32), "task": "go"})
    rec.save_episode()
    rec.stop_image_writer()
    wrist = rec.root / rec.meta.get_video_file_path(0, "observation.images.wrist")
    assert not wrist.exists() and (rec.root / rec.meta.get_video_file_path(0, "observation.images.top")).exists()
    src = tmp_path / "clip.mp4"                               # 30 fps source, 40 frames, brightness = 5 * frame
    wr = cv2.VideoWriter(str(src), cv2.VideoWriter_fourcc(*"mp4v"), 30, (64, 48))
    for i in range(40):
        wr.write(np.full((48, 64, 3), 5 * i, np.uint8))
    wr.release()
    with pytest.raises(ValueError, match="not a video feature"):
        rec.attach_video(0, "observation.state", src)
    with pytest.raises(ValueError, match="does not exist"):
        rec.attach_video(3, "observation.images.wrist", src)
    out = rec.attach_video(0, "observation.images.wrist", src)
    assert out == wrist and wrist.exists() and rec.attach_video(0, "observation.images.wrist", src) == wrist
    rec.update_video_info()
    meta = LeRobotDatasetMetadata("local/toy", root=tmp_path / "toy")
    info = meta.features["observation.images.wrist"]["info"]
    assert info["video.height"] == 48 and info["video.width"] == 64 and round(info["video.fps"]) == 10
    cap = cv2.VideoCapture(str(wrist))
    assert int(cap.get(cv2.CAP_PROP_FRAME_COUNT)) == 8
    cap.release()
    assert rec.encode_episode_videos(0, skip_keys={"observation.images.wrist"}).keys() == {"observation.images.top"}
