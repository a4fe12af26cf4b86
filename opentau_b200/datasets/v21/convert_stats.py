"""Per-episode statistics of a v2.0 dataset directory and the check that they aggregate back to the old dataset-level
statistics (reference ``src/opentau/datasets/v21/convert_stats.py:25-150``).  Video features are sub-sampled (evenly
spaced frames) and therefore compared with a looser tolerance."""

from __future__ import annotations

from pathlib import Path

import numpy as np

from ..compute_stats import aggregate_stats, compute_episode_stats, sample_indices
from ..utils import EPISODES_STATS_PATH, serialize_stats, write_jsonlines


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


def convert_stats(root: str | Path, info: dict, episodes: list[dict], num_workers: int = 0) -> list[dict]:
    """Statistics of every episode (optionally on a thread pool: the work is file reads and numpy reductions), in
    episode order: ``[{"episode_index": i, "stats": {feature: {stat: array}}}]``."""
    root = Path(root)
    if num_workers > 0:
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(max_workers=num_workers) as pool:
            return list(pool.map(lambda ep: episode_stats(root, info, ep), episodes))
    return [episode_stats(root, info, ep) for ep in episodes]


def write_episodes_stats(root: str | Path, rows: list[dict]) -> None:
    write_jsonlines([{"episode_index": r["episode_index"], "stats": serialize_stats(r["stats"])} for r in rows],
                    Path(root) / EPISODES_STATS_PATH)
