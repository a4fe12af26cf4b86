"""Subtask / mistake annotation tools with a scripted vision-language client (no network), on a recorded video dataset."""

import json

import numpy as np
import pyarrow.parquet as pq

from opentau_b200.planner.high_level_planner import CallableClient
from opentau_b200.scripts import add_subtask_response, annotate_mistakes, annotate_subtasks
from test_datasets_cpu import _record


def test_build_response_array_rules():
    subs = [{"time": 0.5, "subtask": "b"}, {"time": 0.0, "subtask": "a"}, {"time": 9.0, "subtask": "late"}]
    out = add_subtask_response.build_response_array(subs, fps=10, length=12)
    assert out == ["a"] * 5 + ["b"] * 7                       # sorted by time; a start beyond the episode is dropped
    assert add_subtask_response.build_response_array([{"time": 0.3, "subtask": "x"}], 10, 5) == ["", "", "", "x", "x"]
    assert add_subtask_response.build_response_array([], 10, 3) == ["", "", ""]


def test_parsers():
    assert annotate_subtasks.parse_json_response('```json\n[{"time": 0, "subtask": "go"}]\n```')[0]["subtask"] == "go"
    assert annotate_subtasks.parse_json_response('Sure! [{"time": 1, "subtask": "x"}] done')[0]["time"] == 1
    assert annotate_subtasks.coerce_subtasks([{"time": "2", "subtask": " b "}, {"time": 0, "subtask": "a"}, {"oops": 1},
                                              {"time": 1, "subtask": ""}]) == [{"time": 0.0, "subtask": "a"},
                                                                              {"time": 2.0, "subtask": "b"}]
    assert annotate_mistakes.parse_success_response('{"success": false, "reason": "dropped"}') is False
    assert annotate_mistakes.parse_success_response("success: TRUE because ...") is True
    assert annotate_mistakes.find_response_runs(["a", "a", "", "b", "b", "b", "a"]) == [(0, 1, "a"), (3, 5, "b"), (6, 6, "a")]


def test_annotate_subtasks_then_mistakes(tmp_path):
    _record(tmp_path / "toy", use_videos=True, episodes=(12, 9))
    root = tmp_path / "toy"
    cfg = tmp_path / "mix.json"
    cfg.write_text(json.dumps({"dataset_mixture": {"datasets": [{"repo_id": "local/toy", "root": str(root)}]}}))
    datasets = annotate_subtasks.load_datasets_from_config(cfg)
    calls = []

    def subtask_model(messages, images):
        calls.append(len(images))
        assert "Frame timestamps" in messages[-1]["content"]
        return 'Here you go:\n```json\n[{"time": 0.0, "subtask": "reach"}, {"time": 0.6, "subtask": "grasp"}]\n```'

    done = annotate_subtasks.run(datasets, CallableClient(subtask_model), sample_fps=5.0, target_size=32)
    assert done == {str(root.resolve()): 2} and calls == [6, 5]              # every 2nd frame of 12 and of 9
    info = json.loads((root / "meta/info.json").read_text())
    assert info["subtask_path"] == annotate_subtasks.SUBTASK_TEMPLATE and info["features"]["response"]["dtype"] == "string"
    resp = pq.read_table(add_subtask_response.episode_parquet(root, info, 0)).column("response").to_pylist()
    assert resp == ["reach"] * 6 + ["grasp"] * 6
    # a second run finds the subtask files and asks nothing
    assert annotate_subtasks.run(datasets, CallableClient(subtask_model), sample_fps=5.0)[str(root.resolve())] == 0
    assert len(calls) == 2

    def judge(messages, images):
        assert len(images) == 1
        failed = "Subtask: grasp" in messages[-1]["content"]
        return json.dumps({"success": not failed, "reason": "scripted"})

    done = annotate_mistakes.run(datasets, CallableClient(judge), target_size=32)
    assert done[str(root.resolve())] == 2
    mist = pq.read_table(add_subtask_response.episode_parquet(root, info, 0)).column("mistake").to_pylist()
    assert mist == [0] * 6 + [1] * 6
    info = json.loads((root / "meta/info.json").read_text())
    assert info["features"]["mistake"]["dtype"] == "int64"
    assert annotate_mistakes.run(datasets, CallableClient(judge))[str(root.resolve())] == 0     # resumable


def test_unusable_answers_leave_no_mistake(tmp_path):
    _record(tmp_path / "toy", use_videos=True, episodes=(6,))
    root = tmp_path / "toy"
    (root / "subtasks").mkdir()
    (root / "subtasks/episode_000000.json").write_text(json.dumps([{"time": 0, "subtask": "only"}]))
    info = json.loads((root / "meta/info.json").read_text())
    info["subtask_path"] = annotate_subtasks.SUBTASK_TEMPLATE
    (root / "meta/info.json").write_text(json.dumps(info))
    assert add_subtask_response.process_dataset(root) == 1
    done = annotate_mistakes.run([{"repo_id": "local/toy", "root": str(root)}], CallableClient(lambda m, i: "no idea"))
    assert done[str(root.resolve())] == 1
    assert pq.read_table(add_subtask_response.episode_parquet(root, info, 0)).column("mistake").to_pylist() == [0] * 6


def test_norm_distribution_flags_stale_metadata(tmp_path):
    """Metadata whose std was inflated by a removed outlier shows up as z_std << 1 and is listed first."""
    from opentau_b200.scripts import diagnose_norm_distribution as dn
    _record(tmp_path / "toy", episodes=(12, 9, 15))
    root = tmp_path / "toy"
    stats = json.loads((root / "meta/stats.json").read_text()) if (root / "meta/stats.json").exists() else None
    rows = dn.run([{"repo_id": "local/toy", "root": str(root)}], tmp_path / "diag")
    fresh = [r for r in rows if r["feature"] == "action"]
    assert len(fresh) == 6 and all(abs(r["z_std"] - 1.0) < 1e-3 and abs(r["z_mean"]) < 1e-6 for r in fresh)
    # make the metadata stale: tenfold std for the state of every episode
    import opentau_b200.datasets.utils as du
    path = root / "meta/episodes_stats.jsonl"
    lines = [json.loads(x) for x in path.read_text().splitlines()]
    for ln in lines:
        ln["stats"]["observation.state"]["std"] = [10 * v for v in ln["stats"]["observation.state"]["std"]]
    path.write_text("\n".join(json.dumps(x) for x in lines) + "\n")
    if stats is not None:
        stats["observation.state"]["std"] = [10 * v for v in stats["observation.state"]["std"]]
        (root / "meta/stats.json").write_text(json.dumps(stats))
    rows = dn.run([{"repo_id": "local/toy", "root": str(root)}], tmp_path / "diag2")
    assert rows[0]["feature"] == "observation.state" and rows[0]["z_std"] < 0.5
    rep = json.loads((tmp_path / "diag2/report.json").read_text())
    assert len(rep["rows"]) == 12 and (tmp_path / "diag2/report.csv").exists()
    fixed = json.loads((tmp_path / "diag2/corrected_stats.json").read_text())
    head = next(iter(fixed))
    assert abs(fixed[head]["observation.state"]["mean"][0] - 17.5) < 1e-6 and du is not None
    a, b = dn.DimStats(2), dn.DimStats(2)
    x = np.random.default_rng(0).normal(size=(50, 2))
    a.update(x[:20], x[:20]), b.update(x[20:], x[20:])
    whole = dn.DimStats(2)
    whole.update(x, x)
    a.merge(b)
    assert np.allclose(a.moments()[1], whole.moments()[1]) and (a.hist == whole.hist).all()


def test_memory_generator_and_nav_planner(tmp_path):
    from PIL import Image
    from opentau_b200.scripts import download_assets, nav_high_level_planner_inference, pi_mem_data_generator as gen
    data = [{"subtask": "open drawer", "success": False, "time": 1.5, "prompt": "tidy up"},
            {"subtask": "open drawer", "success": True, "memory": "kept"}, {"subtask": "pick cup"}]
    path = tmp_path / "segs.json"
    path.write_text(json.dumps(data))
    seen = []

    def model(messages, images):
        seen.append(messages[-1]["content"])
        return f" memory {len(seen)} "

    assert gen.main([str(path), "--skip-existing"], client=CallableClient(model)) == 0
    out = json.loads(path.read_text())
    assert [o["memory"] for o in out] == ["memory 1", "kept", "memory 2"]
    assert "1. [FAILED] (t=1.5s) open drawer" in seen[0] and "Previous memory: (none)" in seen[0]
    assert "Previous memory: kept" in seen[1] and "3. [UNKNOWN] pick cup" in seen[1] and "2. [SUCCESS] open drawer" in seen[1]
    assert gen.main([str(tmp_path / "missing.json")], client=CallableClient(model)) == 1
    frames = tmp_path / "frames"
    frames.mkdir()
    for i in range(3):
        Image.fromarray(np.full((8, 8, 3), 40 * i, np.uint8)).save(frames / f"f{i}.png")
    acts = nav_high_level_planner_inference.main(
        ["--img_path", str(frames)], client=CallableClient(lambda m, i: json.dumps([f"{len(i)} views", "go forward"])))
    assert acts == ["3 views", "go forward"]
    assert download_assets.main(["libero"]) in (2, 3) and download_assets.main(["robocasa"]) in (2, 3)


def test_value_visualizer_pages(tmp_path):
    from opentau_b200.scripts import value_visualizer as vv
    _record(tmp_path / "toy", episodes=(12, 9))
    a = tmp_path / "a.json"
    a.write_text(json.dumps({"(0, 0.0)": -1.0, "(0, 0.5)": -0.5, "(0, 1.1)": 0.0, "1,0.2": 0.3}))
    b = tmp_path / "b.json"
    b.write_text(json.dumps({"0": [{"frame": i, "value": -1 + i / 12, "return": -1 + i / 11} for i in range(12)]}))
    va, vb = vv.load_values(a), vv.load_values(b, fps=10)
    assert [r["t"] for r in va[0]] == [0.0, 0.5, 1.1] and va[1][0]["value"] == 0.3 and vb[0][5]["t"] == 0.5
    pages = vv.render(vb, tmp_path / "viz", dataset_root=tmp_path / "toy", n_frames=4)
    text = pages[0].read_text()
    assert text.count("<img src=\"data:image/jpeg;base64,") == 4 and text.count("<polyline") == 2
    assert len(vv.render(va, tmp_path / "viz2")) == 2


def test_value_visualizer_app_serves_page_episode_and_frames(tmp_path):
    import threading
    import urllib.error
    import urllib.request

    from opentau_b200.scripts import value_visualizer as vv
    from opentau_b200.scripts import value_visualizer_app as app
    _record(tmp_path / "toy", episodes=(12, 9))
    (tmp_path / "dc.json").write_text(json.dumps({"datasets": [{"root": str(tmp_path / "toy"), "episodes": [1, 0]}]}))
    root, repo, eps = app.load_dataset_config(tmp_path / "dc.json")
    assert root == (tmp_path / "toy").resolve() and eps == [0, 1] and repo == "local/dataset"
    b = tmp_path / "b.json"
    b.write_text(json.dumps({"0": [{"frame": i, "value": -1 + i / 12, "return": None} for i in range(12)]}))
    state = app.ViewerState(vv.load_values(b, fps=10), 0, root, fps=10.0)
    assert state.payload["frame"] == list(range(12)) and abs(state.payload["final"] - (-1 + 11 / 12)) < 1e-9
    server = app.make_server(state, port=0)
    th = threading.Thread(target=server.serve_forever, daemon=True)
    th.start()
    base = f"http://127.0.0.1:{server.server_address[1]}"
    try:
        page = urllib.request.urlopen(base + "/", timeout=10).read().decode()
        assert "Timeline" not in page and 'type="range"' in page and "/api/episode" in page
        ep = json.loads(urllib.request.urlopen(base + "/api/episode", timeout=10).read())
        assert ep["episode"] == 0 and len(ep["value"]) == 12 and abs(ep["t"][5] - 0.5) < 1e-9
        jpg = urllib.request.urlopen(base + "/frame/3.jpg", timeout=10).read()
        assert jpg[:2] == b"\xff\xd8" and state.frame_jpeg(3) is jpg or state.frame_jpeg(3) == jpg
        try:
            urllib.request.urlopen(base + "/nothing", timeout=10)
            raise AssertionError("expected 404")
        except urllib.error.HTTPError as e:
            assert e.code == 404
    finally:
        server.shutdown()
        server.server_close()
    import pytest
    with pytest.raises(KeyError):
        app.episode_payload(vv.load_values(b, fps=10), 7, 10.0)


def test_ros_bag_conversion_with_fake_messages(tmp_path):
    """Joint states at 20 Hz, commands at 7 Hz and JPEG frames at 5 Hz are aligned to 10 fps; a broken bag is skipped."""
    import io
    from types import SimpleNamespace as NS

    from PIL import Image

    from opentau_b200.configs.ros2lerobot import RosToLeRobotConfig
    from opentau_b200.configs.types import ROSFeature
    from opentau_b200.datasets.lerobot_dataset import LeRobotDatasetMetadata
    from opentau_b200.scripts.convert_ros_to_lerobot import convert
    from opentau_b200.utils.ros2lerobot import synchronize_sensor_data

    assert synchronize_sensor_data([(0, "a"), (0.26e9, "b"), (0.5e9, "c")], 10, 0.0) == ["a", "a", "b", "b", "c"]
    for name in ("bag_a", "bag_b"):
        (tmp_path / "bags" / name / "recording").mkdir(parents=True)

    def jpeg(v):
        buf = io.BytesIO()
        Image.fromarray(np.full((24, 32, 3), v, np.uint8)).save(buf, format="PNG")
        return buf.getvalue()

    def reader(path):
        if "bag_b" in str(path):
            raise OSError("truncated bag")
        t0 = 100.0
        for i in range(41):                                              # 2 s of joint states at 20 Hz
            t = t0 + i / 20
            stamp = NS(sec=int(t), nanosec=int((t % 1) * 1e9))
            yield "/joint_states", 0, NS(header=NS(stamp=stamp), name=["j2", "j1"], position=[2.0 + i, 1.0 + i],
                                         velocity=[0.2, 0.1])
        for i in range(15):
            yield "/cmd", int((t0 + i / 7) * 1e9), NS(joint_names=["j1", "j2"], motor_cmd=[NS(q=10.0 + i), NS(q=20.0 + i)])
        for i in range(11):
            yield "/cam/compressed", int((t0 + i / 5) * 1e9), NS(data=jpeg(20 * i))

    cfg = RosToLeRobotConfig(
        input_path=str(tmp_path / "bags"), output_path=str(tmp_path / "out"), fps=10, joint_order=["j1", "j2"],
        robot_type="arm", dataset_features={
            "observation.state": ROSFeature("/joint_states", "position", "state", "float32", (4,)),
            "action": ROSFeature("/cmd", "motor_cmd", "action", "float32", (2,)),
            "observation.images.cam": ROSFeature("/cam/compressed", "data", "image", "video", (24, 32, 3))})
    done = convert(cfg, reader=reader, info=lambda p: ("stack the cups", 100.0))
    assert done == {"episodes": 1, "frames": 20, "failed": 1}             # every stream spans 2.0 s: int(2.0 * fps)
    meta = LeRobotDatasetMetadata("out", root=tmp_path / "out")
    assert meta.total_episodes == 1 and meta.total_frames == 20 and meta.tasks[0] == "stack the cups"
    rows = pq.read_table(add_subtask_response.episode_parquet(tmp_path / "out", meta.info, 0)).to_pydict()
    assert np.allclose(rows["observation.state"][0], [1.0, 2.0, 0.1, 0.2])           # reordered to j1, j2; velocities appended
    assert rows["observation.state"][4][0] == 1.0 + 8                     # 0.4 s -> the 20 Hz sample number 8
    assert rows["action"][7] == [15.0, 25.0]                              # 0.7 s -> command number 5


def test_human_video_conversion_with_a_stub_detector(tmp_path):
    import cv2
    from types import SimpleNamespace as NS

    from opentau_b200.datasets.lerobot_dataset import LeRobotDatasetMetadata
    from opentau_b200.scripts.human_video_to_lerobot import convert, landmarks_to_state
    st = landmarks_to_state([[NS(x=1, y=2, z=3), NS(x=4, y=5, z=6)], [NS(x=7, y=8, z=9)]], 12, 6)
    assert st.tolist() == [1, 2, 3, 4, 5, 6, 7, 8, 9, 0, 0, 0]
    assert landmarks_to_state(None, 6, 6).tolist() == [0] * 6
    video = tmp_path / "in.mp4"
    wr = cv2.VideoWriter(str(video), cv2.VideoWriter_fourcc(*"mp4v"), 20.0, (64, 48))
    for i in range(20):
        wr.write(np.full((48, 64, 3), 10 * i, np.uint8))
    wr.release()
    rep = convert(video, tmp_path / "ds", "wave", lambda rgb: np.full(6, rgb[0, 0, 0] / 10.0), 6, fps=10)
    assert rep == {"frames": 10, "fps": 10, "state_dim": 6}
    meta = LeRobotDatasetMetadata("ds", root=tmp_path / "ds")
    rows = pq.read_table(add_subtask_response.episode_parquet(tmp_path / "ds", meta.info, 0)).to_pydict()
    s, a = np.array(rows["observation.state"]), np.array(rows["action"])
    assert np.allclose(a[:-1], s[1:], atol=1e-6) and np.allclose(a[-1], s[-1]) and meta.tasks[0] == "wave"
    assert abs(s[3, 0] - 6.0) < 0.5                                    # every 2nd frame of the 20 fps video


def test_headset_recording_conversion(tmp_path):
    import cv2
    from opentau_b200.datasets.lerobot_dataset import LeRobotDatasetMetadata
    from opentau_b200.scripts import recordhuman_to_lerobot as rh
    # quaternion algebra: a 90 degree turn about z, its inverse and the composition
    qz = np.array([0, 0, np.sin(np.pi / 4), np.cos(np.pi / 4)])
    assert np.allclose(rh.quat_to_rotation_matrix(qz) @ [1, 0, 0], [0, 1, 0], atol=1e-9)
    assert np.allclose(rh.quat_multiply(qz, rh.quat_inverse(qz)), [0, 0, 0, 1], atol=1e-9)
    # a point one metre ahead of a head turned by qz, seen from that head, lies on the camera's own x axis
    cam = rh.world_to_camera(np.array([[0.0, 1.0, 0.0]]), np.zeros(3), qz)
    assert np.allclose(cam, [[1, 0, 0]], atol=1e-9)
    px, py, ok = rh.project_camera_to_pixel(np.array([[0.0, 0.5, 1.0], [0, 0, -1.0]]), 100, 100, 50, 40)
    assert ok.tolist() == [True, False] and px[0] == 50 and py[0] == -10 and np.isnan(px[1])
    video = tmp_path / "rec.mp4"
    wr = cv2.VideoWriter(str(video), cv2.VideoWriter_fourcc(*"mp4v"), 10.0, (64, 48))
    for i in range(10):
        wr.write(np.full((48, 64, 3), 20 * i, np.uint8))
    wr.release()
    ident = [0, 0, 0, 1]
    frames = []
    for i in range(10):
        joints = np.tile(np.array([0.1 * i, 0.0, 1.0] + ident, float), 26)
        frames.append({"t": i / 10, "head_pos": [0.01 * i, 0, 0], "head_rot": ident, "left_joints": joints.tolist(),
                       "left_tracked": True, "right_joints": joints.tolist(), "right_tracked": i % 2 == 0})
    (tmp_path / "rec.json").write_text(json.dumps({"frames": frames}))
    rep = rh.convert(video, tmp_path / "rec.json", tmp_path / "ds", "pick", tracking_origin=(0, 0, 0), eye_offset=0.0,
                     overlay=tmp_path / "overlay.mp4")
    assert rep == {"frames": 10, "fps": 10} and (tmp_path / "overlay.mp4").stat().st_size > 0
    meta = LeRobotDatasetMetadata("ds", root=tmp_path / "ds")
    rows = pq.read_table(add_subtask_response.episode_parquet(tmp_path / "ds", meta.info, 0)).to_pydict()
    s, a = np.array(rows["observation.state"]), np.array(rows["action"])
    assert s.shape == (10, 364) and a.shape == (10, 371)
    assert abs(s[3, 0] - (0.3 - 0.03)) < 1e-5 and s[3, 2] == 1.0          # joint x minus head x, z kept
    assert np.all(s[1, 182:] == 0) and np.any(s[2, 182:] != 0)            # right hand untracked on odd frames
    assert np.allclose(a[:-1, :364], s[1:]) and np.allclose(a[2, 364:], [0.01, 0, 0, 0, 0, 0, 1], atol=1e-6)
    assert np.allclose(a[-1, 364:], [0, 0, 0, 0, 0, 0, 1])
