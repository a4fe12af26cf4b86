"""Online buffer, streaming delta-action statistics, speed buckets."""

import numpy as np
import pytest
import torch

from opentau_b200.datasets.delta_action_stats import HistogramQuantiles, RunningStats, cache_key
from opentau_b200.datasets.online_buffer import OnlineBuffer, compute_sampler_weights
from opentau_b200.datasets.speed_percentiles import episode_speed, speed_buckets


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


def test_speed_buckets_per_task():
    assert episode_speed(np.array([[0.0, 0.0], [3.0, 4.0], [6.0, 8.0]]), fps=2) == 10.0
    speeds = {0: 1.0, 1: 2.0, 2: 3.0, 3: 4.0, 4: 0.5, 5: 9.0}
    tasks = {0: "a", 1: "a", 2: "a", 3: "a", 4: "b", 5: "b"}
    b = speed_buckets(speeds, tasks, n_buckets=2)
    assert [b[i] for i in range(6)] == [1, 1, 2, 2, 1, 2]


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
