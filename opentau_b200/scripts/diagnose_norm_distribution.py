"""CPU diagnostic: distribution of the NORMALISED state / action values, read from the parquet frames themselves.

Every other statistic in a dataset comes from ``meta/stats.json`` / ``episodes_stats.jsonl``; when outliers were removed
from the data but the metadata was never recomputed, those numbers are stale.  This tool streams the real frames of each
dataset of a mixture, normalises them with the METADATA statistics the policy would use, and reports per dimension:
moments and a histogram of ``z = (x - mean) / (std + eps)`` and the data-derived mean / std / min / max next to the
metadata values.  A healthy dimension has ``z_std`` near 1; a dimension whose metadata std was inflated by a since-removed
outlier shows ``z_std << 1`` and ``meta_max >> data_max``.  Same outputs as the reference tool
(``src/opentau/scripts/diagnose_norm_distribution.py:82-702``): ``report.json``, ``report.csv`` and, on request, a
data-derived statistics override; all accumulators are associative, so datasets are processed in parallel and merged.
Figures need matplotlib and are skipped without it.

    python -m opentau_b200.scripts.diagnose_norm_distribution --config mixture.json --output_dir outputs/norm_diag
"""

from __future__ import annotations

import argparse
import csv
import json
import logging
import math
from concurrent.futures import ProcessPoolExecutor
from pathlib import Path

import numpy as np

EPS = 1e-6
_CLIP, _N_LIN, _Z_MAX, _N_LOG = 8.0, 160, 1e5, 30
BEYOND = (3.0, 5.0, 10.0)
log = logging.getLogger(__name__)


def make_bin_edges() -> np.ndarray:
    """Dense linear core in [-8, 8] std, symmetric log-spaced tails to 1e5 std, two open overflow bins."""
    lin = np.linspace(-_CLIP, _CLIP, _N_LIN + 1)
    tail = np.logspace(math.log10(_CLIP), math.log10(_Z_MAX), _N_LOG + 1)[1:]
    return np.concatenate([[-np.inf], -tail[::-1], lin, tail, [np.inf]]).astype(np.float64)


BIN_EDGES = make_bin_edges()
N_BINS = len(BIN_EDGES) - 1


class DimStats:
    """Streaming accumulator for one feature of ``D`` dims: exact raw moments and extremes, plus moments, extremes,
    tail counts and a histogram of the normalised value.  ``merge`` is associative and commutative."""

    def __init__(self, D: int):
        self.D, self.count = D, 0
        z = lambda: np.zeros(D, np.float64)  # noqa: E731
        self.xsum, self.xsq, self.zsum, self.zsq = z(), z(), z(), z()
        self.xmin, self.xmax = np.full(D, np.inf), np.full(D, -np.inf)
        self.zmin, self.zmax = np.full(D, np.inf), np.full(D, -np.inf)
        self.beyond = np.zeros((len(BEYOND), D), np.int64)
        self.hist = np.zeros((D, N_BINS), np.int64)

    def update(self, x: np.ndarray, z: np.ndarray) -> None:
        x, z = x.astype(np.float64), z.astype(np.float64)
        self.count += x.shape[0]
        self.xsum += x.sum(0); self.xsq += (x * x).sum(0)
        self.zsum += z.sum(0); self.zsq += (z * z).sum(0)
        self.xmin = np.minimum(self.xmin, x.min(0)); self.xmax = np.maximum(self.xmax, x.max(0))
        self.zmin = np.minimum(self.zmin, z.min(0)); self.zmax = np.maximum(self.zmax, z.max(0))
        for i, t in enumerate(BEYOND):
            self.beyond[i] += (np.abs(z) > t).sum(0)
        for d in range(self.D):
            self.hist[d] += np.histogram(z[:, d], bins=BIN_EDGES)[0]

    def merge(self, o: "DimStats") -> "DimStats":
        self.count += o.count
        for name in ("xsum", "xsq", "zsum", "zsq", "beyond", "hist"):
            setattr(self, name, getattr(self, name) + getattr(o, name))
        self.xmin, self.xmax = np.minimum(self.xmin, o.xmin), np.maximum(self.xmax, o.xmax)
        self.zmin, self.zmax = np.minimum(self.zmin, o.zmin), np.maximum(self.zmax, o.zmax)
        return self

    def moments(self):
        n = max(self.count, 1)
        xm, zm = self.xsum / n, self.zsum / n
        return xm, np.sqrt(np.maximum(self.xsq / n - xm * xm, 0)), zm, np.sqrt(np.maximum(self.zsq / n - zm * zm, 0))


def normalize(x: np.ndarray, stat: dict, mode: str) -> np.ndarray:
    """The policy's input normalisation (``policies/normalize.py``) restated on numpy rows."""
    g = lambda k: np.asarray(stat[k], np.float64).reshape(-1)  # noqa: E731
    if mode == "MEAN_STD":
        return (x - g("mean")) / (g("std") + EPS)
    if mode == "MIN_MAX":
        return (x - g("min")) / (g("max") - g("min") + EPS) * 2 - 1
    if mode == "QUANTILE":
        return (x - g("q01")) / (g("q99") - g("q01") + EPS) * 2 - 1
    raise ValueError(f"unknown normalisation mode {mode}")


def process_dataset(task: dict) -> dict:
    """One dataset: ``{feature: DimStats}`` for every float vector feature with metadata statistics."""
    import pyarrow.parquet as pq
    from ..datasets.utils import get_version, load_episodes, load_info, load_stats
    root = Path(task["root"])
    info = load_info(root)
    stats = load_stats(root, get_version(info)) or {}
    episodes = sorted(load_episodes(root, get_version(info)))[:task.get("max_episodes")]
    keys = [k for k, f in info["features"].items()
            if f["dtype"] in ("float32", "float64") and len(f["shape"]) == 1 and k in stats and f["shape"][0] > 1
            or k in ("action", "observation.state") and k in stats]
    acc: dict[str, DimStats] = {}
    chunk = int(info.get("chunks_size", 1000))
    for ep in episodes:
        path = root / info["data_path"].format(episode_chunk=ep // chunk, episode_index=ep)
        if not path.is_file():
            continue
        table = pq.read_table(path, columns=[k for k in keys])
        for k in keys:
            x = np.asarray(table.column(k).to_pylist(), np.float64)[::task.get("frame_stride", 1)]
            if x.ndim == 1:
                x = x[:, None]
            acc.setdefault(k, DimStats(x.shape[1])).update(x, normalize(x, stats[k], task.get("norm_mode", "MEAN_STD")))
    return {"head": f"{task['repo_id']}::{info.get('robot_type') or 'unknown'}", "acc": acc,
            "meta": {k: {s: np.asarray(v).reshape(-1).tolist() for s, v in stats[k].items()} for k in keys}}


def finalize(results: list[dict]) -> list[dict]:
    """One row per (head, feature, dim), staleness first (smallest ``z_std``)."""
    rows = []
    for res in results:
        for key, st in res["acc"].items():
            xm, xs, zm, zs = st.moments()
            meta = res["meta"][key]
            for d in range(st.D):
                rows.append({
                    "head": res["head"], "feature": key, "dim": d, "count": st.count,
                    "z_mean": float(zm[d]), "z_std": float(zs[d]), "z_min": float(st.zmin[d]), "z_max": float(st.zmax[d]),
                    **{f"frac_beyond_{int(t)}": float(st.beyond[i, d]) / max(st.count, 1) for i, t in enumerate(BEYOND)},
                    "data_mean": float(xm[d]), "data_std": float(xs[d]), "data_min": float(st.xmin[d]),
                    "data_max": float(st.xmax[d]),
                    **{f"meta_{s}": float(meta[s][d]) for s in ("mean", "std", "min", "max") if s in meta}})
    return sorted(rows, key=lambda r: r["z_std"])


def corrected_stats(results: list[dict]) -> dict:
    out = {}
    for res in results:
        for key, st in res["acc"].items():
            xm, xs, _, _ = st.moments()
            out.setdefault(res["head"], {})[key] = {"mean": xm.tolist(), "std": xs.tolist(), "min": st.xmin.tolist(),
                                                    "max": st.xmax.tolist(), "count": [st.count]}
    return out


def run(datasets: list[dict], output_dir: str | Path, num_workers: int = 0, frame_stride: int = 1,
        max_episodes_per_dataset: int | None = None, norm_mode: str = "MEAN_STD",
        emit_corrected_stats: bool = True) -> list[dict]:
    tasks = [{"repo_id": d.get("repo_id", "local"), "root": d["root"], "frame_stride": frame_stride,
              "max_episodes": max_episodes_per_dataset, "norm_mode": norm_mode} for d in datasets]
    if num_workers > 1 and len(tasks) > 1:
        with ProcessPoolExecutor(num_workers) as ex:
            results = list(ex.map(process_dataset, tasks))
    else:
        results = [process_dataset(t) for t in tasks]
    merged: dict[str, dict] = {}
    for r in results:                                    # datasets that share a head merge into one accumulator
        m = merged.setdefault(r["head"], {"head": r["head"], "acc": {}, "meta": r["meta"]})
        for k, st in r["acc"].items():
            m["acc"][k] = m["acc"][k].merge(st) if k in m["acc"] else st
    results = list(merged.values())
    rows = finalize(results)
    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "report.json").write_text(json.dumps({"bin_edges": BIN_EDGES[1:-1].tolist(), "rows": rows,
                                                 "histograms": {f"{r['head']}/{k}": st.hist.tolist()
                                                                for r in results for k, st in r["acc"].items()}}))
    if rows:
        with open(out / "report.csv", "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=list(rows[0]))
            w.writeheader()
            w.writerows(rows)
    if emit_corrected_stats:
        (out / "corrected_stats.json").write_text(json.dumps(corrected_stats(results), indent=1))
    return rows


def main(argv: list[str] | None = None) -> None:
    from .annotate_subtasks import load_datasets_from_config
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", required=True)
    ap.add_argument("--output_dir", default="outputs/norm_diag")
    ap.add_argument("--num_workers", type=int, default=0)
    ap.add_argument("--frame_stride", type=int, default=1)
    ap.add_argument("--max_episodes_per_dataset", type=int, default=None)
    ap.add_argument("--norm_mode", default="MEAN_STD", choices=["MEAN_STD", "MIN_MAX", "QUANTILE"])
    ap.add_argument("--no_corrected_stats", action="store_true")
    ap.add_argument("--top_n", type=int, default=40)
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO)
    rows = run(load_datasets_from_config(a.config), a.output_dir, a.num_workers, a.frame_stride,
               a.max_episodes_per_dataset, a.norm_mode, not a.no_corrected_stats)
    for r in rows[:a.top_n]:
        print(f"{r['head']:40s} {r['feature']:24s} dim {r['dim']:3d}  z_std {r['z_std']:.3f}  z_max {r['z_max']:.1f}  "
              f"data_max {r['data_max']:.4g}  meta_max {r.get('meta_max', float('nan')):.4g}")


if __name__ == "__main__":
    main()
