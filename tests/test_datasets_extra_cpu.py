"""Online buffer, streaming delta-action statistics, speed buckets."""

import numpy as np
import pytest
import torch

from opentau_b200.datasets.delta_action_stats import HistogramQuantiles, RunningStats, cache_key
from opentau_b200.datasets.online_buffer import OnlineBuffer, compute_sampler_weights
from opentau_b200.datasets import speed_percentiles as SP


def _episode(n, fps=10):
    return {"index": np.arange(n), "frame_index": np.arange(n), "episode_index": np.zeros(n, np.int64),
            "timestamp": np.arange(n) / fps, "observation.state": np.arange(n, dtype=np.float32)[:, None].repeat(2, 1),
            "action": np.ones((n, 2), np.float32)}


def test_online_buffer_fifo_and_delta_queries(tmp_path):
    spec = {"observation.state": {"dtype": "float32", "shape": (2,)}, "action": {"dtype": "float32", "shape": (2,)}}
    buf = OnlineBuffer(tmp_path / "b", spec, buffer_capacity=10, fps=10,
                       delta_timestamps={"observation.state": [-0.1, 0.0], "action": [0.0, 0.1, 0.2]})
    buf.add_data(_episode(4))
    buf.add_data(_episode(4))
    assert len(buf) == 8 and buf.num_episodes == 2
    it = buf[5]                                           # second episode, frame 1
    assert it["episode_index"].item() == 1 and it["observation.state"][:, 0].tolist() == [0.0, 1.0]
    assert it["action_is_pad"].tolist() == [False, False, False]
    assert buf[7]["action_is_pad"].tolist() == [False, True, True]
    buf.add_data(_episode(4))                             # wraps: overwrites the oldest two frames
    assert len(buf) == 10 and buf.num_episodes == 3
    reopened = OnlineBuffer(tmp_path / "b", spec, buffer_capacity=10, fps=10)
    assert len(reopened) == 10
    with pytest.raises(ValueError, match="reserved"):
        OnlineBuffer(tmp_path / "c", {"_x": {"dtype": "float32", "shape": ()}}, 4)

    class Off:
        episode_data_index = {"from": torch.tensor([0, 5]), "to": torch.tensor([5, 10])}
        def __len__(self): return 10
    w = compute_sampler_weights(Off(), 1, buf, 0.25, 0)
    assert w.shape == (20,) and abs(float(w[10:].sum()) - 0.25) < 1e-6 and float(w[4]) == 0.0 and float(w[9]) == 0.0


def test_streaming_stats_equal_batch_stats():
    rng = np.random.default_rng(0)
    x = rng.normal(2.0, 3.0, size=(5000, 3))
    rs = RunningStats(3)
    for part in np.array_split(x, 17):
        rs.update(part)
    r = rs.result()
    np.testing.assert_allclose(r["mean"], x.mean(0), rtol=1e-6)
    np.testing.assert_allclose(r["std"], x.std(0), rtol=1e-6)
    hq = HistogramQuantiles(r["min"], r["max"])
    hq.update(x)
    np.testing.assert_allclose(hq.quantile(0.99), np.quantile(x, 0.99, axis=0), atol=0.02)
    assert cache_key("a/b", 50, 30.0, {"0": 1}, None) != cache_key("a/b", 50, 30.0, {"0": 2}, None)


def test_speed_labels_from_episode_length_percentiles_per_task(tmp_path, caplog):
    """Length ranking per task: 11 labels between the p5 .. p95 boundaries (a length on a boundary takes the upper
    bucket), the neutral label for tasks with fewer than ten distinct lengths, a persisted file that is trusted as it
    is, rows appended for tasks the file lacks, a staleness warning when episodes were added, unknown task indices
    skipped with one warning."""
    import logging
    lengths = {ep: 100 + 10 * ep for ep in range(20)}
    lengths.update({20: 50, 21: 50, 22: 60})                       # task 1: three episodes, two distinct lengths
    ep2task = {**{ep: 0 for ep in range(20)}, 20: 1, 21: 1, 22: 1}
    pct = SP.compute_task_percentiles({0: [lengths[e] for e in range(20)], 1: [50, 50, 60]})
    assert pct[1] is None and len(pct[0]) == 10 and pct[0] == sorted(pct[0])
    assert SP.bucket_episode_length(10, pct[0]) == 0 and SP.bucket_episode_length(10_000, pct[0]) == 100
    assert SP.bucket_episode_length(pct[0][2], pct[0]) == 30        # == p25 -> upper bucket
    assert SP.bucket_episode_length(123, None) == SP.SPARSE_TASK_BUCKET == 50
    (tmp_path / "meta").mkdir()
    names = {"pick": 0, "place": 1}
    got = SP.load_or_compute_speed_percentiles(tmp_path, lengths, ep2task, names)
    rows = SP.load_jsonlines(tmp_path / SP.SPEED_PERCENTILES_PATH)
    assert got == pct and [r["task_index"] for r in rows] == [0, 1] and rows[0]["n_episodes"] == 20
    assert rows[1]["percentiles"] is None and rows[0]["task"] == "pick"
    labels = SP.speed_bucket_by_episode(list(range(23)) + [99], {**lengths, 99: 5}, ep2task, got)
    assert labels[0] == 0 and labels[19] == 100 and labels[21] == 50 and labels[99] == 50
    # a subset load trusts the file silently; a load with MORE episodes warns and still trusts it
    sub = {e: t for e, t in ep2task.items() if e < 10}
    with caplog.at_level(logging.WARNING):
        assert SP.load_or_compute_speed_percentiles(tmp_path, lengths, sub, names) == pct
        assert "stale" not in caplog.text
        more = {**ep2task, 23: 0}
        assert SP.load_or_compute_speed_percentiles(tmp_path, {**lengths, 23: 7}, more, names) == pct
        assert "stale" in caplog.text
    # a task the file lacks is appended, existing rows stay verbatim
    ep3 = {**ep2task, **{30 + i: 2 for i in range(12)}}
    len3 = {**lengths, **{30 + i: 200 + i for i in range(12)}}
    got3 = SP.load_or_compute_speed_percentiles(tmp_path, len3, ep3, {**names, "push": 2})
    rows3 = SP.load_jsonlines(tmp_path / SP.SPEED_PERCENTILES_PATH)
    assert rows3[:2] == rows and rows3[2]["task_index"] == 2 and got3[0] == pct[0] and len(got3[2]) == 10
    with caplog.at_level(logging.WARNING):
        assert SP.episode_to_task_index({0: 0, 1: 7, 2: 7}, {0, 1}) == {0: 0}
        assert caplog.text.count("task_index=7") == 1


def test_success_role_resolution_chain_and_mistake_polarity():
    import numpy as np
    import torch

    from opentau_b200.datasets.lerobot_dataset import LeRobotDataset
    res = LeRobotDataset._resolve_episode_success
    nm = {"success": "is_episode_successful"}
    # 1. mapped column in the frame, then in the episode record
    assert res({"is_episode_successful": torch.tensor([0.0])}, {"success": True}, nm) is False
    assert res({}, {"is_episode_successful": 1, "success": False}, nm) is True
    # 2. the per-episode mean of the mapped column, thresholded at 0.5
    assert res({}, {}, nm, {"is_episode_successful": {"mean": np.array([0.8])}}) is True
    assert res({}, {}, nm, {"is_episode_successful": {"mean": [0.2]}}) is False
    # 3. the plain per-episode key; nothing at all -> None (unlabelled, not failed)
    assert res({}, {"success": np.bool_(False)}, {}) is False and res({}, {}, nm) is None
    cnt = LeRobotDataset._count_success_role_varying_episodes
    stats = {0: {"s": {"min": [0.0], "max": [0.0]}}, 1: {"s": {"min": [0.0], "max": [1.0]}}, 2: {"other": {}}}
    assert cnt(stats, "s") == (1, 2) and cnt([], "s") == (0, 0)

    class Fake:
        meta = type("M", (), {"version": "v2.1", "episodes_stats": {3: {"done_ok": {"mean": [1.0]}}}})()

        def __init__(self, name_map):
            self._nm = name_map

        def _get_name_map(self):
            return self._nm

        _resolve_episode_success = staticmethod(LeRobotDataset._resolve_episode_success)

    attach = LeRobotDataset._attach_mistake_raw
    item = {"mistake": torch.tensor(True)}
    assert attach(Fake({}), item, {"success": True}, 0) is True and item["mistake_raw"] is True     # the column wins
    item = {}
    assert attach(Fake({}), item, {"success": False}, 0) is False and item["mistake_raw"] is True   # inverted success
    item = {}
    assert attach(Fake({"success": "done_ok"}), item, {}, 3) is True and item["mistake_raw"] is False
    item = {}
    assert attach(Fake({}), item, {}, 0) is None and "mistake_raw" not in item
    item = {"oops": torch.tensor([0])}
    assert attach(Fake({"mistake": "oops"}), item, {}, 0) is None and item["mistake_raw"] is False


def test_video_backend_selection_tolerance_and_resample(tmp_path, caplog):
    """Backend probing falls back in order and warns once; every query must lie within the tolerance of a decoded
    frame; a clip is re-timed and trimmed to an exact frame count."""
    import logging
    import numpy as np
    import pytest
    import torch
    from opentau_b200.datasets import video_utils as vu
    from opentau_b200.scripts.eval import write_video
    assert vu.get_safe_default_codec() in vu.BACKENDS
    assert vu.resolve_backend(None) == vu.get_safe_default_codec()
    with pytest.raises(ValueError, match="Unsupported video backend"):
        vu.resolve_backend("gstreamer")
    if vu._probe_backend("torchcodec") is not None:
        vu._warn_downgrade.cache_clear()
        with caplog.at_level(logging.WARNING):
            a = vu.resolve_backend("torchcodec")
            b = vu.resolve_backend("torchcodec")
        assert a == b == vu.get_safe_default_codec()
        assert sum("was requested but cannot load" in r.message for r in caplog.records) == 1     # once per process
    frames = np.stack([np.full((32, 48, 3), 10 * i, np.uint8) for i in range(20)])
    src = tmp_path / "src.mp4"
    write_video(src, frames, 10)
    got = vu.decode_video_frames(src, [0.0, 0.5, 1.9], tolerance_s=0.04, backend="opencv")
    assert got.shape == (3, 3, 32, 48) and abs(float(got[1].mean()) * 255 - 50) < 6
    with pytest.raises(vu.FrameTimestampError):
        vu.decode_video_frames(src, [0.55], tolerance_s=0.01, backend="opencv")
    idx = vu._check_tolerance(torch.tensor([0.1, 0.31]), torch.tensor([0.0, 0.1, 0.2, 0.3]), 0.02, "x")
    assert idx.tolist() == [1, 3]
    with pytest.raises(vu.FrameTimestampError, match="farther than tolerance_s"):
        vu._check_tolerance(torch.tensor([0.16]), torch.tensor([0.0, 0.1, 0.2]), 0.02, "x")
    assert vu.get_video_pixel_channels("yuv420p") == 3 and vu.get_video_pixel_channels("gray16le") == 1
    assert vu.get_video_pixel_channels("yuva420p") == 4
    with pytest.raises(ValueError):
        vu.get_video_pixel_channels("bayer")
    from PIL import Image
    assert vu.get_image_pixel_channels(Image.new("RGBA", (2, 2))) == 4
    out = tmp_path / "out.mp4"
    vu.resample_and_trim_video(src, out, target_fps=5, num_frames=6, start_time=0.4)
    info = vu.get_video_info(out)
    assert info["video.num_frames"] == 6 and abs(info["video.fps"] - 5) < 0.01
    first = vu.decode_video_frames(out, [0.0], 0.05, backend="opencv")
    assert abs(float(first.mean()) * 255 - 40) < 6                        # source frame 4 (0.4 s at 10 fps)
    with pytest.raises(ValueError, match="too short"):
        vu.resample_and_trim_video(src, tmp_path / "o2.mp4", target_fps=10, num_frames=40)
    vu.close_all()


def test_timestamp_sync_and_episode_buffer_validation(tmp_path):
    import pytest

    from opentau_b200.datasets.utils import check_timestamps_sync, validate_episode_buffer
    ts = np.concatenate([np.arange(5) / 10.0, np.arange(4) / 10.0])          # two episodes, clocks restart
    ep = np.array([0] * 5 + [1] * 4)
    index = {"to": np.array([5, 9])}
    assert check_timestamps_sync(ts, ep, index, fps=10, tolerance_s=1e-4)
    dropped = ts.copy()
    dropped[7:] += 0.1                                                        # a frame missing inside episode 1
    assert check_timestamps_sync(dropped, ep, index, 10, 1e-4, raise_value_error=False) is False
    with pytest.raises(ValueError, match="episode_index': 1"):
        check_timestamps_sync(dropped, ep, index, 10, 1e-4)
    assert check_timestamps_sync(dropped, ep, index, 10, 0.2)                 # a looser tolerance accepts it
    with pytest.raises(ValueError, match="same shape"):
        check_timestamps_sync(ts, ep[:-1], index, 10, 1e-4)
    feats = {"action": {}, "observation.images.top": {}, "timestamp": {}, "episode_index": {}}
    good = {"size": 2, "task": ["a", "a"], "episode_index": 3, "action": [], "observation.images.top": [], "timestamp": []}
    validate_episode_buffer(good, 3, feats)
    with pytest.raises(NotImplementedError):
        validate_episode_buffer(good, 4, feats)
    with pytest.raises(ValueError, match="add one or several frames"):
        validate_episode_buffer({**good, "size": 0}, 3, feats)
    late = {k: v for k, v in good.items() if k != "observation.images.top"}
    with pytest.raises(ValueError, match="missing"):
        validate_episode_buffer(late, 3, feats)
    validate_episode_buffer(late, 3, feats, deferred_features={"observation.images.top"})
    with pytest.raises(ValueError, match="task key"):
        validate_episode_buffer({k: v for k, v in good.items() if k != "task"}, 3, feats)
    # the recorder refuses an episode whose clock skipped
    from opentau_b200.datasets.lerobot_dataset import LeRobotDataset
    rec = LeRobotDataset.create("local/skip", fps=10, root=tmp_path / "skip", features={
        "action": {"dtype": "float32", "shape": (2,), "names": None}}, use_videos=False)
    for t in (0.0, 0.1, 0.3):
        rec.add_frame({"action": np.zeros(2, np.float32), "task": "x", "timestamp": t})
    with pytest.raises(ValueError, match="dropped or duplicated"):
        rec.save_episode()


def test_image_writer_threads_and_processes(tmp_path):
    import pytest
    from PIL import Image

    from opentau_b200.datasets.image_writer import AsyncImageWriter, safe_stop_image_writer
    rng = np.random.default_rng(0)
    for label, kw in (("threads", dict(num_processes=0, num_threads=3)), ("procs", dict(num_processes=2, num_threads=2))):
        w = AsyncImageWriter(**kw)
        frames = [rng.integers(0, 255, (24, 32, 3), dtype=np.uint8) for _ in range(12)]
        for i, f in enumerate(frames):
            w.save_image(f if i % 2 else torch.from_numpy(f).permute(2, 0, 1), tmp_path / label / f"frame_{i:03d}.png")
        w.wait_until_done()
        got = sorted((tmp_path / label).glob("*.png"))
        assert len(got) == 12 and np.array_equal(np.asarray(Image.open(got[5])), frames[5])
        w.stop()
        w.stop()                                                            # idempotent
        assert all(not p.is_alive() for p in w.processes)

    class Session:
        def __init__(self):
            self.image_writer = AsyncImageWriter(num_threads=1)

    @safe_stop_image_writer
    def record(dataset):
        raise KeyboardInterrupt

    s = Session()
    with pytest.raises(KeyboardInterrupt):
        record(s)
    assert s.image_writer._stopped


def test_feature_name_registry_is_control_mode_aware():
    import pytest

    from opentau_b200.datasets import standard_data_format_mapping as m
    assert m.feature_mapping_key("org/arm", "ee") == "org/arm::ee"
    for cm in (None, "", "  ", "Unknown"):
        assert m.feature_mapping_key("org/arm", cm) == "org/arm"
    try:
        m.register_mapping("org/arm", {"actions": "action_joint", "state": "s"}, "joint")
        m.register_mapping("org/arm", {"actions": "action_ee", "state": "s"}, "ee")
        m.register_mapping("org/arm", {"actions": "action", "state": "s"})
        assert m.resolve_feature_mapping("org/arm", "joint")["actions"] == "action_joint"
        assert m.resolve_feature_mapping("org/arm", "ee")["actions"] == "action_ee"
        assert m.resolve_feature_mapping("org/arm", "torque")["actions"] == "action"       # falls back to the plain entry
        feats = {"observation.state": {"dtype": "float32"}, "action": {"dtype": "float32"}}
        assert m.get_mapping("org/arm", feats, control_mode="ee")["actions"] == "action_ee"
        assert m.get_mapping("org/arm", feats, {"actions": "mine"})["actions"] == "mine"     # the entry's own map wins
        assert m.get_mapping("nobody/unlisted", feats)["actions"] == "action"                 # inferred
        with pytest.raises(KeyError, match="No feature mapping"):
            m.resolve_feature_mapping("nobody/unlisted", "ee")
    finally:
        for k in ("org/arm", "org/arm::ee", "org/arm::joint"):
            m.DATA_FEATURES_NAME_MAPPING.pop(k, None)
    assert m.DATA_FEATURES_NAME_MAPPING["lerobot/droid_100"]["camera0"].startswith("observation.images.")
