"""Feature statistics: per-episode records and their weighted aggregation
(reference ``src/opentau/datasets/compute_stats.py:30-549``).

Each record holds ``min / max / mean / std / count`` (and, when asked, quantiles ``q01 / q99``) per feature; images
are reduced per channel to shape ``(C,1,1)`` from a sample of frames in [0,1].  Aggregation is exact for
min/max/mean/std (parallel-variance formula) and count-weighted for quantiles.
"""

from __future__ import annotations

import numpy as np


def estimate_num_samples(n: int, min_num: int = 100, max_num: int = 10_000, power: float = 0.75) -> int:
    if n < min_num:
        min_num = n
    return max(min_num, min(int(n ** power), max_num))


def sample_indices(n: int) -> list[int]:
    k = estimate_num_samples(n)
    return np.round(np.linspace(0, n - 1, k)).astype(int).tolist()


def get_feature_stats(array: np.ndarray, axis, keepdims: bool, quantiles: bool = False) -> dict[str, np.ndarray]:
    a = np.asarray(array, dtype=np.float64)
    out = {"min": a.min(axis=axis, keepdims=keepdims), "max": a.max(axis=axis, keepdims=keepdims),
           "mean": a.mean(axis=axis, keepdims=keepdims), "std": a.std(axis=axis, keepdims=keepdims),
           "count": np.array([a.shape[0]])}
    if quantiles:
        out["q01"] = np.quantile(a, 0.01, axis=axis, keepdims=keepdims)
        out["q99"] = np.quantile(a, 0.99, axis=axis, keepdims=keepdims)
    return out


def compute_episode_stats(episode: dict[str, np.ndarray], features: dict[str, dict], quantiles: bool = False) -> dict:
    """``episode[key]``: ``(T, ...)`` arrays; image features are ``(T, C, H, W)`` floats in [0,1] (already sampled)."""
    stats = {}
    for key, data in episode.items():
        ft = features.get(key)
        if ft is None or ft["dtype"] == "string":
            continue
        if ft["dtype"] in ("image", "video"):
            s = get_feature_stats(np.asarray(data), axis=(0, 2, 3), keepdims=True, quantiles=False)
            stats[key] = {k: (v if k == "count" else np.squeeze(v, axis=0)) for k, v in s.items()}
        else:
            arr = np.asarray(data)
            if arr.ndim == 1:
                arr = arr[:, None]
            stats[key] = get_feature_stats(arr, axis=0, keepdims=False, quantiles=quantiles)
    return stats


def _assert_type_and_shape(stats_list: list[dict]) -> None:
    for st in stats_list:
        for fkey, d in st.items():
            for k, v in d.items():
                if not isinstance(v, np.ndarray):
                    raise ValueError(f"stats must be numpy arrays, got {type(v)} for {fkey}.{k}")
                if k == "count" and v.shape != (1,):
                    raise ValueError(f"'count' of {fkey} must have shape (1,), got {v.shape}")


def aggregate_feature_stats(items: list[dict[str, np.ndarray]]) -> dict[str, np.ndarray]:
    means = np.stack([s["mean"] for s in items]).astype(np.float64)
    variances = np.stack([s["std"] for s in items]).astype(np.float64) ** 2
    counts = np.stack([s["count"] for s in items]).astype(np.float64)
    total = counts.sum(axis=0)
    w = counts
    while w.ndim < means.ndim:
        w = np.expand_dims(w, -1)
    mean = (means * w).sum(axis=0) / total
    delta = means - mean
    var = ((variances + delta ** 2) * w).sum(axis=0) / total
    out = {"min": np.min(np.stack([s["min"] for s in items]), axis=0),
           "max": np.max(np.stack([s["max"] for s in items]), axis=0),
           "mean": mean, "std": np.sqrt(var), "count": total.astype(np.int64)}
    for q in ("q01", "q99"):
        if all(q in s for s in items):
            out[q] = (np.stack([s[q] for s in items]) * w).sum(axis=0) / total
    return out


def aggregate_stats(stats_list: list[dict]) -> dict:
    """Merges per-episode (or per-dataset) statistics into one record per feature."""
    _assert_type_and_shape(stats_list)
    keys = {k for st in stats_list for k in st}
    return {k: aggregate_feature_stats([st[k] for st in stats_list if k in st]) for k in keys}
