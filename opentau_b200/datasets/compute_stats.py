"""Feature statistics: per-episode records and their weighted aggregation
(reference ``src/opentau/datasets/compute_stats.py:30-549``).

Each record holds ``min / max / mean / std / count`` (and, when asked, quantiles ``q01 / q99``) per feature; images
are reduced per channel to shape ``(C,1,1)`` from a sample of frames in [0,1].  Aggregation is exact for
min/max/mean/std (parallel-variance formula) and count-weighted for quantiles; a contributor that is non-finite at
some dim is left out AT THAT DIM only, and a quantile that not every contributor carries is dropped, never
back-filled from min / max.
"""

from __future__ import annotations

import logging
import warnings

import numpy as np

#: per-dim quantiles a record may carry (QUANTILE normalisation reads q01 / q99; the rest are diagnostics)
QUANTILE_STAT_NAMES: tuple[str, ...] = ("q01", "q10", "q50", "q90", "q99")


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


def _masked_weighted_mean(values: np.ndarray, weights: np.ndarray, bad: np.ndarray) -> np.ndarray:
    """Per-dim weighted mean over axis 0 that leaves out the entries flagged ``bad``; NaN where nothing is left."""
    w = np.where(bad, 0.0, weights).astype(np.float64)
    total = w.sum(axis=0)
    return np.divide((np.where(bad, 0.0, values) * w).sum(axis=0), total,
                     out=np.full(total.shape, np.nan, np.float64), where=total > 0)


def aggregate_feature_stats(items: list[dict[str, np.ndarray]], weights: list[float] | None = None,
                            contributor_names: list[str] | None = None, context: str | None = None) -> dict[str, np.ndarray]:
    """One feature over several contributors (episodes, or datasets that share a normalisation head).

    ``weights`` REPLACE the contributors' ``count`` (pooling datasets by their frame totals, say).  A contributor whose
    ``mean`` is NaN / Inf at a dim is left out of the mean at that dim; it is left out of the variance where its mean
    OR its std is non-finite; a dim that is non-finite in every contributor stays NaN for the loader to report.
    ``count`` is the plain sum.  Quantiles are the weight-averaged quantiles of the contributors (pooled quantiles
    cannot be recovered exactly; the average is robust to one contributor's extremes, unlike min / max) and appear in
    the result only if EVERY contributor has them: mixing a true q01 with somebody's min would widen the band by
    exactly the outliers that quantile normalisation exists to ignore.  Partial coverage is logged with the names of
    the contributors that lack the quantile."""
    for label, par in (("weights", weights), ("contributor_names", contributor_names)):
        if par is not None and len(par) != len(items):
            raise ValueError(f"{label} ({len(par)}) must be parallel to the statistics list ({len(items)}): a misaligned "
                             "list would silently skew every weighted statistic")
    means = np.stack([np.asarray(s["mean"], np.float64) for s in items])
    variances = np.stack([np.asarray(s["std"], np.float64) for s in items]) ** 2
    counts = (np.stack([np.asarray(w, np.float64).reshape(1) for w in weights]) if weights is not None
              else np.stack([np.asarray(s["count"], np.float64) for s in items]))
    total = counts.sum(axis=0)
    w = counts
    while w.ndim < means.ndim:
        w = np.expand_dims(w, -1)
    mean_bad, var_bad = ~np.isfinite(means), ~np.isfinite(variances)
    mean = _masked_weighted_mean(means, w, mean_bad)
    spread = np.where(var_bad, 0.0, variances) + np.where(mean_bad, 0.0, means - mean) ** 2
    var = _masked_weighted_mean(spread, w, var_bad | mean_bad)
    mins = np.stack([np.asarray(s["min"], np.float64) for s in items])
    maxs = np.stack([np.asarray(s["max"], np.float64) for s in items])
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", category=RuntimeWarning)          # all-NaN slices stay NaN on purpose
        out = {"min": np.nanmin(np.where(np.isfinite(mins), mins, np.nan), axis=0),
               "max": np.nanmax(np.where(np.isfinite(maxs), maxs, np.nan), axis=0),
               "mean": mean, "std": np.sqrt(var),
               "count": total.astype(np.int64) if weights is None else total}
    lacking: dict[tuple[int, ...], list[str]] = {}
    for q in QUANTILE_STAT_NAMES:
        have = [q in s for s in items]
        if not any(have):
            continue
        if not all(have):
            lacking.setdefault(tuple(i for i, h in enumerate(have) if not h), []).append(q)
            continue
        vals = np.stack([np.asarray(s[q], np.float64) for s in items])
        out[q] = _masked_weighted_mean(vals, w, ~np.isfinite(vals))
    for missing, names in lacking.items():
        who = [contributor_names[i] if contributor_names else f"#{i}" for i in missing]
        logging.warning("%squantile(s) %s dropped from the aggregate: %d of %d contributor(s) do not carry them (%s%s); "
                        "recompute their statistics with quantiles to enable quantile normalisation",
                        f"{context}: " if context else "", names, len(missing), len(items), who[:10],
                        ", ..." if len(who) > 10 else "")
    return out


def aggregate_stats(stats_list: list[dict], weights: list[float] | None = None,
                    contributor_names: list[str] | None = None, context: str | None = None) -> dict:
    """Merges per-episode (or per-dataset) statistics into one record per feature (union of the features; a feature
    that some contributors lack is pooled over those that have it, with the parallel lists narrowed alike)."""
    _assert_type_and_shape(stats_list)
    for label, par in (("weights", weights), ("contributor_names", contributor_names)):
        if par is not None and len(par) != len(stats_list):
            raise ValueError(f"{label} ({len(par)}) must be parallel to stats_list ({len(stats_list)})")
    out = {}
    for key in sorted({k for st in stats_list for k in st}):
        present = [i for i, st in enumerate(stats_list) if key in st]
        out[key] = aggregate_feature_stats(
            [stats_list[i][key] for i in present],
            None if weights is None else [weights[i] for i in present],
            contributor_names=None if contributor_names is None else [contributor_names[i] for i in present],
            context=f"{context}, feature {key!r}" if context else f"feature {key!r}")
    return out
