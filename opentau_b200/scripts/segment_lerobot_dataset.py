"""Cut the episodes of a LeRobot dataset into one episode per subtask segment
(reference ``src/opentau/scripts/segment_lerobot_dataset.py``).

Reads ``segments`` of every episode (segment start frames, see ``attach_metadata``; ``[start, end)`` pairs work too), and writes a new v2.1 dataset
whose episodes are the segments; the task of a new episode is the segment's ``response`` text when present, else the
original task.  Image features are carried over (videos are re-encoded per new episode).
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import numpy as np


def segment(src_ds, out_root: str | Path, repo_id: str) -> dict:
    from ..datasets.lerobot_dataset import LeRobotDataset
    from ..datasets.utils import DEFAULT_FEATURES
    feats = {k: dict(v) for k, v in src_ds.meta.features.items() if k not in DEFAULT_FEATURES and k != "response"}
    use_videos = bool(src_ds.meta.video_keys)
    rec = LeRobotDataset.create(repo_id, src_ds.fps, root=out_root, robot_type=src_ds.meta.robot_type, features=feats,
                                use_videos=use_videos, image_writer_threads=2 if use_videos else 0)
    was, was_delta = src_ds.standardize, src_ds.delta_timestamps
    src_ds.standardize, src_ds.delta_timestamps = False, {}      # raw single frames, no action chunks / history
    n_new = 0
    try:
        for ep in src_ds.episodes:
            length = int(src_ds.meta.episodes[ep]["length"])
            raw = src_ds.meta.episodes[ep].get("segments") or [0]
            # start frames (each segment runs to the next start, the last to the episode's end); explicit
            # [start, end) pairs are accepted as well
            starts = [int(x[0]) if isinstance(x, (list, tuple)) else int(x) for x in raw]
            ends = [int(x[1]) if isinstance(x, (list, tuple)) and len(x) > 1 else (starts[i + 1] if i + 1 < len(starts)
                                                                                    else length)
                    for i, x in enumerate(raw)]
            segs = list(zip(starts, ends))
            base = int(src_ds.episode_data_index["from"][src_ds.epi2idx[ep]])
            for s, e in segs:
                for fi in range(int(s), int(e)):
                    item = src_ds[base + fi]
                    frame = {"task": item.get("response") or item["task"]}
                    for k, ft in feats.items():
                        v = item[k]
                        if ft["dtype"] in ("image", "video"):
                            v = (v.permute(1, 2, 0).float().clamp(0, 1).numpy() * 255).astype(np.uint8)
                        elif ft["dtype"] != "string":
                            v = np.asarray(v, dtype=ft["dtype"]).reshape(ft["shape"])
                        frame[k] = v
                    rec.add_frame(frame)
                rec.save_episode()
                n_new += 1
    finally:
        src_ds.standardize, src_ds.delta_timestamps = was, was_delta
        rec.stop_image_writer()
    return {"source_episodes": len(src_ds.episodes), "segments": n_new}


def main(argv=None) -> None:
    from ..configs.default import DatasetConfig, DatasetMixtureConfig
    from ..configs.train import TrainPipelineConfig
    from ..datasets.factory import make_dataset
    ap = argparse.ArgumentParser()
    ap.add_argument("--repo-id", required=True)
    ap.add_argument("--root", required=True)
    ap.add_argument("--out-root", required=True)
    ap.add_argument("--out-repo-id", default=None)
    a = ap.parse_args(argv)
    dc = DatasetConfig(repo_id=a.repo_id, root=a.root)
    ds = make_dataset(dc, TrainPipelineConfig(dataset_mixture=DatasetMixtureConfig(datasets=[dc])))
    print(json.dumps(segment(ds, a.out_root, a.out_repo_id or f"{a.repo_id}_segments")))


if __name__ == "__main__":
    main()
