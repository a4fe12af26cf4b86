"""Codebase v2.0 -> v2.1: per-episode statistics (``meta/episodes_stats.jsonl``) replace the dataset-level
``meta/stats.json`` (reference ``src/opentau/datasets/v21/convert_dataset_v20_to_v21.py``)."""

from __future__ import annotations

import argparse
from pathlib import Path

import numpy as np

from ..compute_stats import compute_episode_stats
from ..utils import (EPISODES_PATH, EPISODES_STATS_PATH, INFO_PATH, STATS_PATH, load_info, load_jsonlines, serialize_stats,
                     write_json, write_jsonlines)


def convert(root: str | Path, delete_old_stats: bool = False) -> int:
    import pyarrow.parquet as pq
    root = Path(root)
    info = load_info(root)
    if str(info["codebase_version"]).lstrip("v") != "2.0":
        raise ValueError(f"expected a v2.0 dataset, found {info['codebase_version']}")
    rows = []
    for ep in load_jsonlines(root / EPISODES_PATH):
        i = int(ep["episode_index"])
        path = root / info["data_path"].format(episode_chunk=i // info.get("chunks_size", 1000), episode_index=i)
        t = pq.read_table(path)
        data = {}
        for k, ft in info["features"].items():
            if ft["dtype"] in ("image", "video", "string") or k not in t.column_names:
                continue
            col = t.column(k).to_numpy(zero_copy_only=False)
            data[k] = np.stack([np.asarray(x) for x in col]) if col.dtype == object else col
        rows.append({"episode_index": i, "stats": serialize_stats(compute_episode_stats(data, info["features"]))})
    write_jsonlines(rows, root / EPISODES_STATS_PATH)
    info["codebase_version"] = "v2.1"
    info["features"] = {k: {**v, "shape": list(v["shape"])} for k, v in info["features"].items()}
    write_json(info, root / INFO_PATH)
    if delete_old_stats and (root / STATS_PATH).exists():
        (root / STATS_PATH).unlink()
    return len(rows)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--root", required=True)
    ap.add_argument("--delete-old-stats", action="store_true")
    a = ap.parse_args(argv)
    print(f"converted {convert(a.root, a.delete_old_stats)} episodes")


if __name__ == "__main__":
    main()
