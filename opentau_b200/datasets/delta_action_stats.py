"""Statistics of DELTA actions (``a[t+i] - state[t]`` on mapped dims) over a dataset
(reference ``src/opentau/datasets/delta_action_stats.py:60-857``).

The stats stored with a dataset describe absolute actions.  When ``use_delta_joint_actions`` is on, normalisation
needs the statistics of the transformed targets, which depend on the action-chunk length and frequency, so they are
computed here by streaming over (a subsample of) the frames: exact running min / max / mean / variance
(Chan's parallel update) and quantiles from fixed-range histograms refined in a second pass.

Two entry points:

* :func:`compute_delta_stats_from_columns` / :func:`load_or_compute_delta_stats`: the training path.  It works on the
  numeric ``state`` / ``action`` columns alone (no image or video is decoded), gathers each anchor frame's chunk with
  the same clipping and resampling as the dataset's ``__getitem__`` (frames past the episode end repeat the last row and
  are KEPT: training marks them padded but still normalises them), subtracts the anchor's state on the mapped dims,
  and caches the result under the dataset's own ``meta/delta_action_stats/`` keyed by everything that changes it.
  The main process computes; the other ranks poll the file system for the file (no collective, so a long first pass
  cannot run into a process-group timeout).
* :func:`compute_delta_action_stats`: the same numbers from the items of any dataset object (slow; used by tools).
"""

from __future__ import annotations

import contextlib
import hashlib
import json
import logging
import os
import time
import uuid
from pathlib import Path
from typing import Sequence

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


# ---------------------------------------------------------------------------------------------------------------------
# column-based pass (no decode) with a per-dataset cache
# ---------------------------------------------------------------------------------------------------------------------
CACHE_SUBDIR = Path("meta") / "delta_action_stats"
CACHE_VERSION = 1                 # bump when the payload or the semantics change: older files are then ignored
POLL_TIMEOUT_S = 3 * 60 * 60      # the pass is O(frames x chunk) per dataset and runs once per configuration
POLL_INTERVAL_S = 5.0
_READONLY_WARNED: set[str] = set()


def delta_stats_cache_key(*, state_index: Sequence[int] | None, action_index: Sequence[int] | None,
                          delta_map: dict | None, chunk_offsets: Sequence[float], vector_resample_strategy: str,
                          episodes: Sequence[int] | None, excluded_episodes: Sequence[int] | None, fps: float | None,
                          revision: str | None, max_rows: int | None = None) -> str:
    """12 hex digits over everything that separates two configurations of ONE dataset (its root supplies identity).
    Offsets and fps are rounded so float noise cannot split the cache; ``max_rows`` enters only when set, so the
    expensive uncapped file keeps its name."""
    payload = {
        "version": CACHE_VERSION,
        "state_index": None if state_index is None else [int(i) for i in state_index],
        "action_index": None if action_index is None else [int(i) for i in action_index],
        "delta_map": sorted(normalize_delta_map(delta_map).items()),
        "chunk_offsets": [round(float(o), 6) for o in chunk_offsets],
        "vector_resample_strategy": vector_resample_strategy,
        "episodes": None if episodes is None else sorted(int(e) for e in episodes),
        "excluded_episodes": None if excluded_episodes is None else sorted(int(e) for e in excluded_episodes),
        "fps": None if fps is None else round(float(fps), 6),
        "revision": revision,
    }
    if max_rows is not None:
        payload["max_rows"] = int(max_rows)
    return hashlib.sha256(json.dumps(payload, sort_keys=True, separators=(",", ":")).encode()).hexdigest()[:12]


def gather_chunks(values: np.ndarray, anchors: np.ndarray, offsets: np.ndarray, ep_start: int, ep_end: int,
                  strategy: str) -> np.ndarray:
    """``(len(anchors), len(offsets), dim)``: rows ``anchor + offset`` clipped into the episode ``[ep_start, ep_end)``,
    by rounding (``nearest``) or by interpolation between the two neighbouring rows (``linear``)."""
    soft = np.clip(anchors[:, None] + offsets[None, :], ep_start, ep_end - 1)
    if strategy == "nearest":
        return values[np.rint(soft).astype(np.int64)]
    if strategy == "linear":
        lo = np.floor(soft).astype(np.int64)
        frac = soft - lo
        hi = np.clip(lo + (frac > 0.0), ep_start, ep_end - 1)
        return values[lo] + frac[..., None] * (values[hi] - values[lo])
    raise ValueError(f"unknown vector_resample_strategy {strategy!r}: use 'nearest' or 'linear'")


def select_anchor_rows(spans: Sequence[tuple[int, int]], max_rows: int | None) -> list[tuple[np.ndarray, int, int]]:
    """Anchor rows per episode span ``(start, end)``.  Under a cap ONE stride runs across the concatenated spans
    (not a prefix: later episodes may be the ones that widen the range; and not restarted per episode: that would
    put an anchor on every episode's first frame).  ``ceil(total / stride) <= max_rows``, so the cap is hard.  The
    true bounds travel with the rows because clipping still needs them."""
    total = sum(hi - lo for lo, hi in spans)
    if max_rows is None or total <= max_rows:
        return [(np.arange(lo, hi, dtype=np.int64), lo, hi) for lo, hi in spans if hi > lo]
    stride = -(-total // max_rows)
    out, seen = [], 0
    for lo, hi in spans:
        rows = np.arange(lo + (-seen) % stride, hi, stride, dtype=np.int64)
        seen += hi - lo
        if rows.size:
            out.append((rows, lo, hi))
    return out


def _finish(rs: RunningStats, hq: "HistogramQuantiles") -> dict[str, np.ndarray]:
    out = rs.result()
    out["q01"], out["q99"] = hq.quantile(0.01), hq.quantile(0.99)
    out["count"] = np.asarray(out["count"], np.int64).reshape(1)
    return out


def compute_delta_stats_from_columns(states: np.ndarray, actions: np.ndarray, episode_index: np.ndarray, *,
                                     delta_map: dict | None, chunk_offsets: Sequence[float],
                                     state_index: Sequence[int] | None = None,
                                     action_index: Sequence[int] | None = None, strategy: str = "nearest",
                                     episodes: set[int] | None = None, max_rows: int | None = None,
                                     block_frames: int = 65536) -> dict[str, dict[str, np.ndarray]]:
    """``{"actions": {...}, "state": {...}}`` in POST-INDEX space from the stored columns (rows ordered by episode).

    Pass 1 finds the range of the deltas so the histogram edges are fixed up front (an edge that moves while an
    episode-ordered stream widens the range smears the quantiles); pass 2 accumulates moments and histograms.  The
    state statistics use the same anchors, so both features describe one sample set."""
    states = np.asarray(states, np.float64)
    actions = np.asarray(actions, np.float64)
    episode_index = np.asarray(episode_index, np.int64)
    if states.ndim != 2 or actions.ndim != 2 or len(states) != len(actions) or len(states) == 0:
        raise ValueError(f"state / action columns must be (rows, dim) of equal length, got {states.shape} / {actions.shape}")
    if state_index is not None:
        states = states[:, list(state_index)]
    if action_index is not None:
        actions = actions[:, list(action_index)]
    dm = normalize_delta_map(delta_map)
    a_pos = np.array(sorted(dm), np.int64)
    s_pos = np.array([dm[int(a)] for a in a_pos], np.int64)
    offsets = np.asarray(chunk_offsets, np.float64)
    cuts = np.flatnonzero(np.diff(episode_index)) + 1
    starts, ends = np.concatenate(([0], cuts)), np.concatenate((cuts, [len(episode_index)]))
    spans = [(int(lo), int(hi)) for lo, hi in zip(starts, ends) if episodes is None or int(episode_index[lo]) in episodes]
    anchors = select_anchor_rows(spans, max_rows)
    if not anchors:
        raise ValueError("no frame of the selected episodes is present in the columns")

    def blocks():
        for rows, lo, hi in anchors:
            for b in range(0, len(rows), block_frames):
                fr = rows[b:b + block_frames]
                chunk = gather_chunks(actions, fr.astype(np.float64), offsets, lo, hi, strategy)
                if a_pos.size:
                    chunk[:, :, a_pos] -= states[fr][:, None, s_pos]     # one state per chunk, broadcast over the horizon
                yield chunk.reshape(-1, chunk.shape[-1])

    lo_v, hi_v = np.full(actions.shape[1], np.inf), np.full(actions.shape[1], -np.inf)
    for flat in blocks():
        lo_v, hi_v = np.minimum(lo_v, flat.min(0)), np.maximum(hi_v, flat.max(0))
    rs, hq = RunningStats(actions.shape[1]), HistogramQuantiles(lo_v, hi_v, bins=5000)
    for flat in blocks():
        rs.update(flat)
        hq.update(flat)
    st_rows = states[np.concatenate([rows for rows, _, _ in anchors])]
    srs, shq = RunningStats(states.shape[1]), HistogramQuantiles(st_rows.min(0), st_rows.max(0), bins=5000)
    srs.update(st_rows)
    shq.update(st_rows)
    if rs.n < 2 or srs.n < 2:
        raise ValueError(f"cannot compute statistics from {rs.n} action / {srs.n} state sample(s)")
    return {"actions": _finish(rs, hq), "state": _finish(srs, shq)}


def _serialize(stats: dict[str, dict[str, np.ndarray]]) -> str:
    return json.dumps({"version": CACHE_VERSION,
                       "stats": {f: {k: np.asarray(v).tolist() for k, v in d.items()} for f, d in stats.items()}})


def _deserialize(text: str) -> dict[str, dict[str, np.ndarray]] | None:
    """``None`` for anything that is not a complete payload of the current version (the caller recomputes)."""
    try:
        data = json.loads(text)
        if data.get("version") != CACHE_VERSION:
            return None
        return {f: {k: np.asarray(v, np.int64 if k == "count" else np.float32) for k, v in d.items()}
                for f, d in data["stats"].items()}
    except Exception:  # noqa: BLE001 - a torn or foreign file is a cache miss
        return None


def _atomic_write_text(text: str, path: Path) -> None:
    tmp = path.with_suffix(f"{path.suffix}.{uuid.uuid4().hex}.tmp")
    try:
        tmp.write_text(text)
        os.replace(tmp, path)
    finally:
        if tmp.exists():
            with contextlib.suppress(OSError):
                tmp.unlink()


def _wait_for_file(path: Path, timeout_s: float, interval_s: float) -> dict[str, dict[str, np.ndarray]] | None:
    deadline, last_log = time.monotonic() + timeout_s, time.monotonic()
    while time.monotonic() < deadline:
        if path.is_file():
            got = _deserialize(path.read_text())
            if got is not None:
                return got
        if time.monotonic() - last_log > 120.0:
            last_log = time.monotonic()
            logging.info("waiting for the main process to write %s", path)
        time.sleep(interval_s)
    return None


def load_or_compute_delta_stats(root: str | Path, cache_key: str, compute, *, timeout_s: float = POLL_TIMEOUT_S,
                                interval_s: float = POLL_INTERVAL_S) -> dict[str, dict[str, np.ndarray]]:
    """The cached statistics under ``root/meta/delta_action_stats/<key>.json``, or ``compute()``'s result (written
    there by the main process).  Other ranks poll for the file; if the directory cannot be written (a read-only
    dataset mount) every rank computes for itself, with one warning per root, because no file will ever appear."""
    from ..parallel import control
    path = Path(root) / CACHE_SUBDIR / f"{cache_key}.json"
    if path.is_file():
        got = _deserialize(path.read_text())
        if got is not None:
            return got
    writable = True
    try:
        path.parent.mkdir(parents=True, exist_ok=True)
        writable = os.access(path.parent, os.W_OK)
    except OSError:
        writable = False
    if not writable:
        if str(root) not in _READONLY_WARNED:
            _READONLY_WARNED.add(str(root))
            logging.warning("%s is not writable: delta-action statistics are recomputed by every process of every run",
                            path.parent)
        return compute()
    if control.is_main_process():
        stats = compute()
        try:
            _atomic_write_text(_serialize(stats), path)
        except OSError as exc:
            logging.warning("could not cache delta-action statistics at %s (%s)", path, exc)
        return stats
    got = _wait_for_file(path, timeout_s, interval_s)
    if got is None:
        logging.warning("no delta-action statistics appeared at %s within %.0f s; computing them in this process",
                        path, timeout_s)
        return compute()
    return got
