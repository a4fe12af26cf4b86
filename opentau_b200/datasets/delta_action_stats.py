"""Statistics of DELTA actions (``a[t+i] - state[t]`` on mapped dims) over a dataset
(reference ``src/opentau/datasets/delta_action_stats.py:60-857``).

The stats stored with a dataset describe absolute actions.  When ``use_delta_joint_actions`` is on, normalisation
needs the statistics of the transformed targets, which depend on the action-chunk length and frequency, so they are
computed here by streaming over (a subsample of) the frames: exact running min / max / mean / variance
(Chan's parallel update) and quantiles from fixed-range histograms refined in a second pass.  Rank 0 computes and
caches (key = dataset + chunk + delta map + row cap), the other ranks wait at a barrier and read the cache.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path

import numpy as np

from .action_indexing import normalize_delta_map


class RunningStats:
    """Streaming min / max / mean / std over rows of width ``d`` (numerically stable chunk merge)."""

    def __init__(self, d: int):
        self.n = 0
        self.mean = np.zeros(d, np.float64)
        self.m2 = np.zeros(d, np.float64)
        self.min = np.full(d, np.inf)
        self.max = np.full(d, -np.inf)

    def update(self, x: np.ndarray) -> None:
        x = np.asarray(x, np.float64).reshape(-1, self.mean.shape[0])
        if len(x) == 0:
            return
        n_b, mean_b = len(x), x.mean(0)
        m2_b = ((x - mean_b) ** 2).sum(0)
        delta = mean_b - self.mean
        tot = self.n + n_b
        self.mean = self.mean + delta * n_b / tot
        self.m2 = self.m2 + m2_b + delta ** 2 * self.n * n_b / tot
        self.n = tot
        self.min, self.max = np.minimum(self.min, x.min(0)), np.maximum(self.max, x.max(0))

    def result(self) -> dict[str, np.ndarray]:
        std = np.sqrt(self.m2 / max(self.n, 1))
        return {"min": self.min.astype(np.float32), "max": self.max.astype(np.float32), "mean": self.mean.astype(np.float32),
                "std": std.astype(np.float32), "count": np.array([self.n])}


class HistogramQuantiles:
    """Per-dimension quantiles from ``bins`` equal-width buckets between known min and max (error <= one bucket)."""

    def __init__(self, lo: np.ndarray, hi: np.ndarray, bins: int = 4096):
        self.lo, self.hi, self.bins = lo.astype(np.float64), np.maximum(hi, lo + 1e-12).astype(np.float64), bins
        self.hist = np.zeros((len(lo), bins), np.int64)

    def update(self, x: np.ndarray) -> None:
        x = np.asarray(x, np.float64).reshape(-1, len(self.lo))
        idx = np.clip(((x - self.lo) / (self.hi - self.lo) * self.bins).astype(np.int64), 0, self.bins - 1)
        for d in range(len(self.lo)):
            self.hist[d] += np.bincount(idx[:, d], minlength=self.bins)

    def quantile(self, q: float) -> np.ndarray:
        cdf = np.cumsum(self.hist, axis=1)
        tot = cdf[:, -1:]
        k = (cdf >= q * tot).argmax(axis=1)
        return (self.lo + (k + 0.5) / self.bins * (self.hi - self.lo)).astype(np.float32)


def cache_key(repo_id: str, chunk: int, action_freq: float, delta_map: dict, max_rows: int | None, version: str = "1") -> str:
    blob = json.dumps([repo_id, chunk, action_freq, sorted(normalize_delta_map(delta_map).items()), max_rows, version])
    return hashlib.sha256(blob.encode()).hexdigest()[:16]


def compute_delta_action_stats(dataset, max_rows: int | None = None, quantiles: bool = True, seed: int = 0) -> dict:
    """``dataset[i]`` must return the standard item (``actions (T, A)`` already delta-transformed, ``action_is_pad``)."""
    n = len(dataset)
    rows = np.arange(n) if not max_rows or max_rows >= n else np.sort(np.random.default_rng(seed).choice(n, max_rows, replace=False))
    A = int(dataset[int(rows[0])]["real_action_dim"])
    rs = RunningStats(A)
    kept = []
    for i in rows:
        it = dataset[int(i)]
        a = it["actions"].float().numpy()[:, :A]
        a = a[~it["action_is_pad"].numpy()]
        rs.update(a)
        if quantiles:
            kept.append(a)
    out = rs.result()
    if quantiles:
        hq = HistogramQuantiles(rs.min, rs.max)
        for a in kept:
            hq.update(a)
        out["q01"], out["q99"] = hq.quantile(0.01), hq.quantile(0.99)
    return out


def get_or_compute_delta_action_stats(dataset, cache_dir: str | Path, repo_id: str, chunk: int, action_freq: float,
                                      delta_map: dict, max_rows: int | None = None) -> dict:
    from ..parallel import control
    f = Path(cache_dir) / f"delta_action_stats_{cache_key(repo_id, chunk, action_freq, delta_map, max_rows)}.json"
    if control.is_main_process() and not f.exists():
        st = compute_delta_action_stats(dataset, max_rows)
        f.parent.mkdir(parents=True, exist_ok=True)
        f.write_text(json.dumps({k: np.asarray(v).tolist() for k, v in st.items()}))
    control.wait_for_everyone()
    return {k: np.asarray(v, np.float32 if k != "count" else np.int64) for k, v in json.loads(f.read_text()).items()}
