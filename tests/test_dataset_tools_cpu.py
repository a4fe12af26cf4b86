"""Dataset tooling: metadata attachment -> subgoal frames and responses, segmentation, visualisation, v2.0 -> v2.1
conversion, token-length scan, checkpoint extraction."""

import json

import numpy as np
import torch

from opentau_b200.configs.default import DatasetConfig, DatasetMixtureConfig
from opentau_b200.configs.train import TrainPipelineConfig
from opentau_b200.datasets.factory import make_dataset, make_dataset_mixture
from opentau_b200.datasets.lerobot_dataset import LeRobotDatasetMetadata
from opentau_b200.scripts.attach_metadata import attach
from opentau_b200.scripts.segment_lerobot_dataset import segment
from opentau_b200.scripts.visualize_dataset import visualize_episode
from test_datasets_cpu import _record


def _cfg(root, **mix):
    dc = DatasetConfig(repo_id="local/toy", root=str(root))
    return dc, TrainPipelineConfig(dataset_mixture=DatasetMixtureConfig(datasets=[dc], action_freq=10.0, **mix),
                                   resolution=(56, 56), num_cams=1, action_chunk=5, batch_size=2, dataloader_batch_size=2)


def test_attach_segment_and_visualize(tmp_path):
    _record(tmp_path / "toy", episodes=(10, 8))
    out = attach(tmp_path / "toy", {"episodes": {"0": {"quality": 4, "success": True, "speed": 2,
                                                        "segments": [[0, 4, "reach"], [4, 10, "grasp"]]},
                                                 "1": {"success": False}}})
    assert out == {"episodes": 2, "frames_labelled": 10}
    meta = LeRobotDatasetMetadata("local/toy", root=tmp_path / "toy")
    assert meta.episodes[0]["segments"] == [0, 4] and meta.episodes[1]["success"] is False
    dc, cfg = _cfg(tmp_path / "toy", subgoal_drop_prob=0.0, subgoal_end_of_segment_prob=1.0, response_drop_prob=0.0,
                   metadata_drop_all_prob=0.0, metadata_drop_each_prob=0.0)
    ds = make_dataset(dc, cfg)
    s = ds[1]
    assert s["response"] == "reach" and ds[6]["response"] == "grasp" and ds[12]["response"] == ""
    assert s["subgoal0"].shape == (3, 56, 56) and not bool(s["subgoal_is_pad"])
    assert abs(float(s["subgoal0"][0, 28, 28]) * 255 - 9) < 2            # frame 3 = end of the first segment
    assert int(s["quality"]) == 4 and int(s["speed"]) == 2
    rep = segment(ds, tmp_path / "seg", "local/toy_seg")
    assert rep == {"source_episodes": 2, "segments": 3}
    seg_meta = LeRobotDatasetMetadata("local/toy_seg", root=tmp_path / "seg")
    assert [seg_meta.episodes[i]["length"] for i in range(3)] == [4, 6, 8]
    assert seg_meta.tasks[0] == "reach" and seg_meta.tasks[1] == "grasp"
    summ = visualize_episode(ds, 0, tmp_path / "viz", n_frames=4)
    assert summ["length"] == 10 and len(summ["files"]) == 3 and all((tmp_path / "viz" / f).exists() for f in summ["files"])


def test_convert_v20_to_v21_and_token_scan(tmp_path):
    from opentau_b200.datasets.v21.convert_dataset_v20_to_v21 import convert
    from opentau_b200.scripts.compute_max_token_length import scan
    from opentau_b200.utils.tokenizer import DctActionTokenizer, load_text_tokenizer
    _record(tmp_path / "toy", episodes=(6, 6))
    root = tmp_path / "toy"
    info = json.loads((root / "meta/info.json").read_text())
    info["codebase_version"] = "v2.0"
    (root / "meta/info.json").write_text(json.dumps(info))
    (root / "meta/episodes_stats.jsonl").unlink()
    assert convert(root) == 2
    meta = LeRobotDatasetMetadata("local/toy", root=root)
    assert meta.version == "v2.1" and np.allclose(meta.stats["observation.state"]["max"], 11.0)
    dc, cfg = _cfg(root)
    mix = make_dataset_mixture(cfg)
    out = scan(mix, load_text_tokenizer("none", 1024), DctActionTokenizer(256), max_samples=8)
    assert out["prompt"]["max"] >= 2 and out["discrete_actions"]["n"] == 8


def test_extract_reasoner_keys():
    from opentau_b200.scripts.extract_cosmos3_reasoner import extract
    st = {"reasoner.model.language_model.layers.0.w": torch.zeros(1), "generator.x": torch.zeros(1)}
    out = extract(st)
    assert list(out) == ["model.qwen3vl_with_expert.backbone.model.language_model.layers.0.w"]


def _write_v16(root, n_eps=3, ep_len=5, with_col=False):
    """A codebase-v1.6 directory: sharded parquet, flat metadata, safetensors statistics."""
    import json

    import numpy as np
    import pyarrow as pa
    import pyarrow.parquet as pq
    from safetensors.numpy import save_file

    (root / "data").mkdir(parents=True)
    (root / "meta_data").mkdir()
    rows = {"observation.state": [], "action": [], "episode_index": [], "frame_index": [], "timestamp": [],
            "index": [], "next.done": []}
    if with_col:
        rows["language_instruction"] = []
    i = 0
    for e in range(n_eps):
        for f in range(ep_len):
            rows["observation.state"].append([float(i), float(e), 0.5])
            rows["action"].append([float(f), -1.0])
            rows["episode_index"].append(e)
            rows["frame_index"].append(f)
            rows["timestamp"].append(f / 10.0)
            rows["index"].append(i)
            rows["next.done"].append(f == ep_len - 1)
            if with_col:
                rows["language_instruction"].append(
                    "tf.Tensor(b'open the drawer', shape=(), dtype=string)" if e < 2 else "close the drawer")
            i += 1
    t = pa.table({k: pa.array(v, type=pa.list_(pa.float32())) if k in ("observation.state", "action") else pa.array(v)
                  for k, v in rows.items()})
    half = t.num_rows // 2
    pq.write_table(t.slice(0, half), root / "data" / "train-00000-of-00002.parquet")
    pq.write_table(t.slice(half), root / "data" / "train-00001-of-00002.parquet")
    (root / "meta_data" / "info.json").write_text(json.dumps({"fps": 10, "video": False}))
    st = np.asarray(rows["observation.state"], dtype=np.float32)
    save_file({"observation.state/mean": st.mean(0), "observation.state/std": st.std(0),
               "observation.state/min": st.min(0), "observation.state/max": st.max(0)},
              str(root / "meta_data" / "stats.safetensors"))
    return st


def test_convert_v16_to_v20_then_v21(tmp_path):
    import json

    import numpy as np
    import pyarrow.parquet as pq

    from opentau_b200.datasets.utils import load_jsonlines
    from opentau_b200.datasets.v2.convert_dataset_v1_to_v2 import batch_convert, convert_dataset
    from opentau_b200.datasets.v21.convert_dataset_v20_to_v21 import convert

    st = _write_v16(tmp_path / "v1")
    info = convert_dataset(tmp_path / "v1", tmp_path / "v2", single_task="stack the cubes", robot_type="so101",
                           motor_names={"action": ["shoulder", "gripper"]})
    assert info["codebase_version"] == "v2.0" and info["total_episodes"] == 3 and info["total_frames"] == 15
    assert info["features"]["action"]["names"] == {"motors": ["shoulder", "gripper"]}
    assert info["features"]["observation.state"]["shape"] == [3] and info["video_path"] is None
    eps = load_jsonlines(tmp_path / "v2" / "meta" / "episodes.jsonl")
    assert [e["length"] for e in eps] == [5, 5, 5] and eps[1]["tasks"] == ["stack the cubes"]
    t = pq.read_table(tmp_path / "v2" / "data" / "chunk-000" / "episode_000001.parquet")
    assert t.num_rows == 5 and set(t.column("task_index").to_pylist()) == {0}
    assert t.column("index").to_pylist() == list(range(5, 10))
    stats = json.loads((tmp_path / "v2" / "meta" / "stats.json").read_text())
    np.testing.assert_allclose(stats["observation.state"]["mean"], st.mean(0), rtol=1e-6)
    # the v2.0 result is a valid input of the next converter
    assert convert(tmp_path / "v2") == 3
    assert json.loads((tmp_path / "v2" / "meta" / "info.json").read_text())["codebase_version"] == "v2.1"

    # tasks from a column (Open-X tensor reprs are cleaned), and the batch driver that survives a bad job
    _write_v16(tmp_path / "v1c", with_col=True)
    status = batch_convert([
        {"v1_dir": tmp_path / "v1c", "v2_dir": tmp_path / "v2c", "single_task": "ignored: the column wins"},
        {"v1_dir": tmp_path / "missing", "v2_dir": tmp_path / "v2x", "single_task": "x"},
    ], log_path=tmp_path / "log.txt")
    assert status[str(tmp_path / "v1c")] == "converted" and status[str(tmp_path / "missing")].startswith("failed")
    tasks = load_jsonlines(tmp_path / "v2c" / "meta" / "tasks.jsonl")
    assert [x["task"] for x in tasks] == ["open the drawer", "close the drawer"]
    eps = load_jsonlines(tmp_path / "v2c" / "meta" / "episodes.jsonl")
    assert eps[2]["tasks"] == ["close the drawer"]
    t = pq.read_table(tmp_path / "v2c" / "data" / "chunk-000" / "episode_000002.parquet")
    assert "language_instruction" not in t.column_names and set(t.column("task_index").to_pylist()) == {1}
    assert len((tmp_path / "log.txt").read_text().splitlines()) >= 2


def test_convert_v20_to_v21_workers_check_metadata_fix_and_batch(tmp_path):
    from opentau_b200.datasets.compute_stats import aggregate_stats
    from opentau_b200.datasets.utils import load_episodes_stats, serialize_stats
    from opentau_b200.datasets.v21.convert_dataset_v20_to_v21 import batch_convert, convert, fix_language_instruction
    import pytest

    def back_to_v20(root, wrong_stats=False):
        agg = aggregate_stats(list(load_episodes_stats(root).values()))
        if wrong_stats:
            agg["observation.state"]["mean"] = agg["observation.state"]["mean"] + 1.0
        (root / "meta/stats.json").write_text(json.dumps(serialize_stats(agg)))
        info = json.loads((root / "meta/info.json").read_text())
        info["codebase_version"] = "v2.0"
        (root / "meta/info.json").write_text(json.dumps(info))
        (root / "meta/episodes_stats.jsonl").unlink()
        return info

    a, b = tmp_path / "a", tmp_path / "b"
    _record(a, episodes=(6, 5))
    _record(b, episodes=(4, 4))
    info = back_to_v20(a)
    # a stale metadata entry that no parquet file holds is repaired; anything else is refused
    info["features"]["language_instruction"] = {"dtype": "string", "shape": [1], "names": None}
    (a / "meta/info.json").write_text(json.dumps(info))
    assert fix_language_instruction(a) == "removed 'language_instruction'"
    assert fix_language_instruction(a) == "skipped (no difference)"
    assert "language_instruction" not in json.loads((a / "meta/info.json").read_text())["features"]
    # threads + the check that the aggregated episode statistics reproduce the old dataset-level ones
    assert convert(a, num_workers=2, check=True, delete_old_stats=True) == 2
    assert not (a / "meta/stats.json").exists()
    assert LeRobotDatasetMetadata("local/toy", root=a).version == "v2.1"
    back_to_v20(b, wrong_stats=True)
    with pytest.raises(AssertionError, match="observation.state"):
        convert(b, check=True)
    status = batch_convert([b, tmp_path / "nope"], log_path=tmp_path / "log.txt")
    assert status[str(b)] == "converted 2 episodes" and status[str(tmp_path / "nope")].startswith("failed")


def test_strict_copy_only_annotation_pipeline(tmp_path):
    import pyarrow.parquet as pq
    import pytest

    from opentau_b200.planner.high_level_planner import CallableClient
    from opentau_b200.scripts.attach_metadata import attach_annotations, load_and_validate_annotations
    _record(tmp_path / "toy", episodes=(10, 8))
    ann = [{"episode_id": 0, "quality": 4, "segments": [{"start": 0, "subtask": "reach", "success": True},
                                                        {"start": 4, "subtask": "grasp", "success": False}]},
           {"episode_id": 1, "quality": 2, "segments": [{"start": 0, "subtask": "place", "success": True}]}]
    before = (tmp_path / "toy" / "meta" / "episodes.jsonl").read_text()
    out = attach_annotations(tmp_path / "toy", ann, tmp_path / "copy", skip_memory=True)
    assert out["episodes"] == 2 and out["frames"] == 18 and out["memory_calls"] == 0
    assert (tmp_path / "toy" / "meta" / "episodes.jsonl").read_text() == before            # the source is never touched
    t = pq.read_table(tmp_path / "copy" / "data/chunk-000/episode_000000.parquet").to_pydict()
    assert t["response"] == ["reach"] * 4 + ["grasp"] * 6 and t["mistake"] == [0] * 4 + [1] * 6
    assert t["memory"][5] == "memory5"
    meta = LeRobotDatasetMetadata("local/toy", root=tmp_path / "copy")
    assert meta.episodes[0]["segments"] == [0, 4] and meta.episodes[0]["quality"] == 4 and meta.episodes[1]["quality"] == 2
    assert meta.features["mistake"]["dtype"] == "int64" and meta.features["memory"]["dtype"] == "string"
    with pytest.raises(FileExistsError):
        attach_annotations(tmp_path / "toy", ann, tmp_path / "copy", skip_memory=True)
    # memories: one model call per segment, asked before anything is written
    seen = []
    client = CallableClient(lambda messages, images: seen.append(messages[-1]["content"]) or f"did {len(seen)} things")
    out = attach_annotations(tmp_path / "toy", ann, tmp_path / "copy", overwrite=True, client=client)
    assert out["memory_calls"] == 3 and "[FAILED]" in seen[1] and "task 0" in seen[0]
    t = pq.read_table(tmp_path / "copy" / "data/chunk-000/episode_000000.parquet").to_pydict()
    assert t["memory"][0] == "did 1 things" and t["memory"][9] == "did 2 things"
    with pytest.raises(ValueError, match="chat client"):
        attach_annotations(tmp_path / "toy", ann, tmp_path / "other")
    assert not (tmp_path / "other").exists()
    # every structural fault is named before any file is written
    lengths = {0: 10, 1: 8}
    good = json.loads(json.dumps(ann))
    cases = [
        (lambda a: a.pop(), "Missing annotations for episodes: \\[1\\]"),
        (lambda a: a.append({**a[0], "episode_id": 7}), "Unknown episodes"),
        (lambda a: a.append(dict(a[0])), "Duplicate episode_id 0"),
        (lambda a: a[0].update(quality=6), "quality must be in 1..5"),
        (lambda a: a[0].update(quality=True), "quality must be int"),
        (lambda a: a[0]["segments"][0].update(start=1), "first segment must start at 0"),
        (lambda a: a[0]["segments"][1].update(start=0), "strictly increase"),
        (lambda a: a[0]["segments"][1].update(start=4.0), "frame index, not a time"),
        (lambda a: a[0]["segments"][1].update(start=10), ">= episode length 10"),
        (lambda a: a[0]["segments"][1].update(success="no"), "success must be bool"),
        (lambda a: a[1].update(segments=[]), "non-empty 'segments'"),
        (lambda a: a[0].pop("quality"), "missing required key 'quality'"),
    ]
    for mutate, message in cases:
        bad = json.loads(json.dumps(good))
        mutate(bad)
        with pytest.raises(ValueError, match=message):
            load_and_validate_annotations(bad, lengths)
    with pytest.raises(ValueError, match="must be a list"):
        load_and_validate_annotations({"episodes": {}}, lengths)
