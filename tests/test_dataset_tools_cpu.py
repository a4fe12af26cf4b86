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
    assert meta.episodes[0]["segments"] == [[0, 4], [4, 10]] and meta.episodes[1]["success"] is False
    dc, cfg = _cfg(tmp_path / "toy", subgoal_drop_prob=0.0, subgoal_end_of_segment_prob=1.0, response_drop_prob=0.0,
                   metadata_drop_all_prob=0.0, metadata_drop_each_prob=0.0)
    ds = make_dataset(dc, cfg)
    s = ds[1]
    assert s["response"] == "reach" and ds[6]["response"] == "grasp" and ds[12]["response"] == ""
    assert s["subgoal0"].shape == (3, 56, 56) and not bool(s["subgoal0_is_pad"])
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
    from opentau_b200.datasets.v2.convert_dataset_v20_to_v21 import convert
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
