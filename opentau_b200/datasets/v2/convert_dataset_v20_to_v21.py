"""Codebase v2.0 -> v2.1: per-episode statistics (``meta/episodes_stats.jsonl``) replace the dataset-level
``meta/stats.json`` (reference ``src/opentau/datasets/v21/convert_dataset_v20_to_v21.py``; per-episode work and the
check against the old statistics ``v21/convert_stats.py:52-150``; the metadata repair
``v21/_remove_language_instruction.py:33-85``; the driver over many datasets
``v21/batch_convert_dataset_v20_to_v21.py``).  Everything works on dataset directories on disk."""

from __future__ import annotations

import argparse
from pathlib import Path

import numpy as np

from ..compute_stats import aggregate_stats, compute_episode_stats, sample_indices
from ..utils import (EPISODES_PATH, EPISODES_STATS_PATH, INFO_PATH, STATS_PATH, load_info, load_jsonlines, serialize_stats,
                     write_json, write_jsonlines)


def fix_language_instruction(root: str | Path) -> str:
    """Some v2.0 exports list a ``language_instruction`` feature in ``meta/info.json`` that no parquet file holds.
    Drop it from the metadata; any other disagreement between metadata and parquet columns is an error."""
    import pyarrow.parquet as pq
    root = Path(root)
    info = load_info(root)
    first = root / info["data_path"].format(episode_chunk=0, episode_index=0)
    in_parquet = set(pq.read_schema(first).names)
    in_meta = {k for k, ft in info["features"].items() if ft["dtype"] != "video"}
    if in_parquet - in_meta:
        raise ValueError(f"in parquet but not in info.json: {sorted(in_parquet - in_meta)}")
    extra = in_meta - in_parquet
    if not extra:
        return "skipped (no difference)"
    if extra != {"language_instruction"}:
        raise ValueError(f"in info.json but not in parquet: {sorted(extra)}")
    info["features"].pop("language_instruction")
    write_json(info, root / INFO_PATH)
    return "removed 'language_instruction'"


def _video_samples(root: Path, info: dict, key: str, ep: int, length: int) -> np.ndarray | None:
    """A sub-sample of one episode's video frames as (n, C, H, W) floats in [0, 1]; None without the file."""
    from ..video_utils import decode_video_frames
    path = root / info["video_path"].format(episode_chunk=ep // info.get("chunks_size", 1000), video_key=key,
                                            episode_index=ep)
    if not path.exists():
        return None
    ts = [i / info["fps"] for i in sample_indices(length)]
    frames = decode_video_frames(path, ts, tolerance_s=1.0 / info["fps"])
    return np.asarray(frames, dtype=np.float32)


def episode_stats(root: Path, info: dict, ep: dict) -> dict:
    import pyarrow.parquet as pq
    i = int(ep["episode_index"])
    path = root / info["data_path"].format(episode_chunk=i // info.get("chunks_size", 1000), episode_index=i)
    t = pq.read_table(path)
    data = {}
    for k, ft in info["features"].items():
        if ft["dtype"] == "video" and info.get("video_path"):
            frames = _video_samples(root, info, k, i, int(ep.get("length", t.num_rows)))
            if frames is not None:
                data[k] = frames
            continue
        if ft["dtype"] in ("image", "video", "string") or k not in t.column_names:
            continue
        col = t.column(k).to_numpy(zero_copy_only=False)
        data[k] = np.stack([np.asarray(x) for x in col]) if col.dtype == object else col
    return {"episode_index": i, "stats": compute_episode_stats(data, info["features"])}


def check_aggregate_stats(rows: list[dict], features: dict, reference: dict, video_tol=(1e-2, 1e-2),
                          default_tol=(5e-6, 6e-5)) -> None:
    """The per-episode statistics, aggregated, must reproduce the old dataset-level statistics (sub-sampled video
    frames get a looser tolerance)."""
    agg = aggregate_stats([r["stats"] for r in rows])
    for key, ft in features.items():
        rtol, atol = video_tol if ft["dtype"] in ("video", "image") else default_tol
        for stat, val in agg.get(key, {}).items():
            if key in reference and stat in reference[key]:
                np.testing.assert_allclose(np.asarray(val, dtype=np.float64).reshape(-1),
                                           np.asarray(reference[key][stat], dtype=np.float64).reshape(-1),
                                           rtol=rtol, atol=atol, err_msg=f"feature='{key}' stats='{stat}'")


def convert(root: str | Path, delete_old_stats: bool = False, num_workers: int = 0, check: bool = False) -> int:
    root = Path(root)
    info = load_info(root)
    if str(info["codebase_version"]).lstrip("v") != "2.0":
        raise ValueError(f"expected a v2.0 dataset, found {info['codebase_version']}")
    episodes = load_jsonlines(root / EPISODES_PATH)
    if num_workers > 0:
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(max_workers=num_workers) as pool:
            rows = list(pool.map(lambda ep: episode_stats(root, info, ep), episodes))
    else:
        rows = [episode_stats(root, info, ep) for ep in episodes]
    if check and (root / STATS_PATH).exists():
        import json
        check_aggregate_stats(rows, info["features"], json.loads((root / STATS_PATH).read_text()))
    rows = [{"episode_index": r["episode_index"], "stats": serialize_stats(r["stats"])} for r in rows]
    write_jsonlines(rows, root / EPISODES_STATS_PATH)
    info["codebase_version"] = "v2.1"
    info["features"] = {k: {**v, "shape": list(v["shape"])} for k, v in info["features"].items()}
    write_json(info, root / INFO_PATH)
    if delete_old_stats and (root / STATS_PATH).exists():
        (root / STATS_PATH).unlink()
    return len(rows)


def batch_convert(roots: list[str | Path], log_path: str | Path | None = None, **kw) -> dict[str, str]:
    """Convert many dataset directories; a failure is recorded and the batch goes on."""
    import traceback
    status: dict[str, str] = {}
    for root in roots:
        try:
            status[str(root)] = f"converted {convert(root, **kw)} episodes"
        except Exception:  # noqa: BLE001
            status[str(root)] = "failed\n    " + traceback.format_exc()
        if log_path:
            with open(log_path, "a") as f:
                f.write(f"{root}: {status[str(root)]}\n")
    return status


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--root", required=True, nargs="+")
    ap.add_argument("--delete-old-stats", action="store_true")
    ap.add_argument("--num-workers", type=int, default=0)
    ap.add_argument("--check", action="store_true", help="aggregated episode statistics must match meta/stats.json")
    ap.add_argument("--fix-language-instruction", action="store_true")
    a = ap.parse_args(argv)
    if a.fix_language_instruction:
        for r in a.root:
            print(f"{r}: {fix_language_instruction(r)}")
    kw = {"delete_old_stats": a.delete_old_stats, "num_workers": a.num_workers, "check": a.check}
    if len(a.root) == 1:
        print(f"converted {convert(a.root[0], **kw)} episodes")
    else:
        for r, st in batch_convert(a.root, **kw).items():
            print(f"{r}: {st.splitlines()[0]}")


if __name__ == "__main__":
    main()
