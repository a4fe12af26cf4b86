"""Fit the discrete action tokenizer (DCT + byte-pair merges) on the action chunks of a dataset mixture, on CPU
(reference ``src/opentau/scripts/fit_fast_tokenizer.py:15-1760``).

The tokenizer is an auxiliary cross-entropy target beside the flow-matching loss; specialising its merge table to the
mixture's own action distribution shortens the token sequences the policy has to predict.  It has to be fitted on
exactly what the policy will hand it at training time, so the pipeline reuses the training pieces:

1. the mixture JSON (``$ref`` includes allowed) becomes a ``DatasetMixtureConfig`` inside a stub pipeline config
   (``num_cams = 0``: no image or video is decoded) and goes through ``make_dataset_mixture``: same column selection,
   delta joint actions, episode selection and normalisation heads as a training run;
2. chunks are drawn per dataset in proportion to the mixture weights, straight from the numeric action columns, at
   offsets ``k / action_freq`` seconds (each dataset's own frame rate when the mixture has no common one), clipped to
   the episode and resampled like ``__getitem__`` does, then zero-padded to ``--action-dim``;
3. every chunk is min-max normalised to ``[-1, 1]`` by the policy's own ``Normalize`` module over the statistics of ITS
   ``(robot_type, control_mode)`` head (``--no-per-head-norm``: one pooled range for everything, which under-spreads
   each head and makes token-length analysis underestimate truncation), with the epsilon and the zero-range
   convention of ``--config-version``;
4. the merge table is learned (native trainer when built), the tokenizer and a sidecar naming the convention are
   written, held-out chunks are round-tripped, and ``fit_report.json`` records inputs, per-dataset counts, per-head
   ranges, token-length percentiles, the share of chunks above ``--max-token-length`` and timings.

    python -m opentau_b200.scripts.fit_fast_tokenizer --mixture-json mix.json --out-dir tok/ --chunk-size 50 \\
        [--total-chunks 1000000] [--action-dim 32] [--vocab-size 2048] [--scale 10] [--pilot] [--no-per-head-norm]
"""

from __future__ import annotations

import argparse
import hashlib
import json
import logging
import time
from pathlib import Path
from typing import Any

import numpy as np

from ..configs.policies import CURRENT_CONFIG_VERSION, LEGACY_EPS, OPENPI_EPS
from ..policies.loading import ACTION_NORM_META_FILE
from ..utils.tokenizer import BpeDctActionTokenizer

TOKENIZER_FILE = "action_tokenizer.json"
REPORT_FILE = "fit_report.json"
PILOT_CHUNKS = 50_000
#: below this many learned merges the vocabulary is mostly the base alphabet: raise --vocab-size
MIN_MERGE_HEADROOM = 100


def parse_args(argv: list[str] | None = None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Fit the DCT + byte-pair action tokenizer on a dataset mixture.",
                                formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    p.add_argument("--mixture-json", type=Path, required=True, help="DatasetMixtureConfig JSON (may use $ref)")
    p.add_argument("--out-dir", type=Path, required=True)
    p.add_argument("--total-chunks", type=int, default=1_000_000)
    p.add_argument("--chunk-size", type=int, required=True, help="action horizon of the policy (steps per chunk)")
    p.add_argument("--action-dim", type=int, default=32, help="the policy's max_action_dim; wider datasets are cut")
    p.add_argument("--max-state-dim", type=int, default=128)
    p.add_argument("--vocab-size", type=int, default=2048)
    p.add_argument("--scale", type=float, default=10.0, help="DCT coefficients are multiplied by this, then rounded")
    p.add_argument("--max-token-length", type=int, default=64,
                   help="the policy's discrete_action_max_length: the report gives the share of chunks above it")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--config-version", type=int, default=CURRENT_CONFIG_VERSION,
                   help="normalisation convention to fit under (0: a zero-range dim maps to -1; >= 1: to 0)")
    p.add_argument("--per-head-norm", dest="per_head_norm", action="store_true", default=True)
    p.add_argument("--no-per-head-norm", dest="per_head_norm", action="store_false",
                   help="one pooled min / max for every dataset (how tokenizers were fitted before heads existed)")
    p.add_argument("--holdout", type=float, default=0.02, help="share of the chunks kept out of the fit for the check")
    p.add_argument("--pilot", action="store_true", help=f"at most {PILOT_CHUNKS} chunks, written to out_dir/pilot/")
    p.add_argument("--skip-fit", action="store_true", help="sampling and normalisation only (timing)")
    p.add_argument("--log-level", default="INFO")
    return p.parse_args(argv)


def parse_mixture(path: Path):
    """``(DatasetMixtureConfig, sha256 of the resolved JSON)``: the hash identifies the data recipe in the report."""
    from ..configs.codec import decode
    from ..configs.default import DatasetMixtureConfig
    from ..configs.refs import load_json_with_refs
    raw = load_json_with_refs(path)
    if isinstance(raw, dict) and "dataset_mixture" in raw:
        raw = raw["dataset_mixture"]
    digest = hashlib.sha256(json.dumps(raw, sort_keys=True, default=str).encode()).hexdigest()
    return decode(DatasetMixtureConfig, raw, "dataset_mixture"), digest


def build_train_cfg(mixture_cfg, *, chunk_size: int, action_dim: int, max_state_dim: int, seed: int):
    """The smallest pipeline config that sends the mixture through the training-time dataset code without cameras."""
    from ..configs.train import TrainPipelineConfig
    return TrainPipelineConfig(dataset_mixture=mixture_cfg, num_cams=0, action_chunk=chunk_size,
                               max_action_dim=action_dim, max_state_dim=max_state_dim, batch_size=1,
                               dataloader_batch_size=1, seed=seed, val_freq=0)


def compute_budgets(weights: list[float], total: int) -> list[int]:
    """Chunks per dataset in proportion to the mixture weights (largest remainders get the leftover units)."""
    w = np.asarray(weights, np.float64)
    if (w < 0).any() or w.sum() <= 0:
        raise ValueError(f"mixture weights must be non-negative with a positive sum, got {weights}")
    exact = w / w.sum() * total
    base = np.floor(exact).astype(np.int64)
    for i in np.argsort(-(exact - base), kind="stable")[: int(total - base.sum())]:
        base[i] += 1
    return base.tolist()


def sample_dataset_chunks(ds, n: int, chunk_size: int, action_freq: float | None, rng: np.random.Generator) -> np.ndarray:
    """``(n, chunk_size, emitted action width)`` from the dataset's numeric columns: anchors drawn uniformly over its
    frames (with replacement only when it has fewer frames than asked for), steps ``k / action_freq`` seconds ahead."""
    from ..datasets.delta_action_stats import gather_chunks
    num = ds._numeric
    names = ds._get_name_map()
    actions = num[names["actions"]].numpy().astype(np.float64)
    episode = num["episode_index"].numpy().astype(np.int64)
    if actions.ndim == 1:
        actions = actions[:, None]
    if ds.action_index is not None:
        actions = actions[:, list(ds.action_index)]
    states = None
    if ds.delta_action_state_map:
        states = num[names["state"]].numpy().astype(np.float64)
        if ds.state_index is not None:
            states = states[:, list(ds.state_index)]
    rows = len(actions)
    anchors = np.sort(rng.choice(rows, size=n, replace=rows < n))
    step = float(ds.fps) / float(action_freq) if action_freq else 1.0
    offsets = np.arange(chunk_size, dtype=np.float64) * step
    cuts = np.flatnonzero(np.diff(episode)) + 1
    starts, ends = np.concatenate(([0], cuts)), np.concatenate((cuts, [rows]))
    which = np.searchsorted(starts, anchors, side="right") - 1
    out = np.empty((n, chunk_size, actions.shape[1]), np.float32)
    for e in np.unique(which):
        sel = np.flatnonzero(which == e)
        fr = anchors[sel]
        chunk = gather_chunks(actions, fr.astype(np.float64), offsets, int(starts[e]), int(ends[e]),
                              ds.vector_resample_strategy)
        if states is not None:
            dm = {int(a): int(b) for a, b in ds.delta_action_state_map.items()}
            a_pos = np.array(sorted(dm), np.int64)
            chunk[:, :, a_pos] -= states[fr][:, None, [dm[int(a)] for a in a_pos]]
        out[sel] = chunk
    return out


def pad_to_action_dim(chunks: np.ndarray, action_dim: int) -> np.ndarray:
    """Zero-pads (or cuts: dims beyond the policy's width never reach it, so they do not belong in the corpus)."""
    n, t, d = chunks.shape
    out = np.zeros((n, t, action_dim), np.float32)
    out[:, :, :min(d, action_dim)] = chunks[:, :, :action_dim]
    return out


def normalize_chunks(chunks: np.ndarray, head_index: np.ndarray, head_stats: list[dict], *, config_version: int,
                     action_dim: int) -> np.ndarray:
    """Min-max normalisation by the policy's own module, so the corpus and the training targets cannot drift apart."""
    import torch

    from ..configs.types import FeatureType, NormalizationMode, PolicyFeature
    from ..policies.normalize import Normalize
    norm = Normalize({"actions": PolicyFeature(FeatureType.ACTION, (action_dim,))}, {"ACTION": NormalizationMode.MIN_MAX},
                     per_dataset_stats=head_stats, zero_range_center=config_version >= 1,
                     eps=OPENPI_EPS if config_version >= 1 else LEGACY_EPS)
    out = np.empty_like(chunks)
    idx = torch.from_numpy(np.asarray(head_index, np.int64))
    for lo in range(0, len(chunks), 65536):
        part = norm({"actions": torch.from_numpy(chunks[lo:lo + 65536])}, idx[lo:lo + 65536])["actions"]
        out[lo:lo + 65536] = part.numpy()
    return out


def pooled_head(head_stats: list[dict]) -> dict:
    """One range over all heads (the legacy global normalisation): outer envelope of the heads' min / max."""
    mins = np.stack([np.asarray(h["actions"]["min"], np.float64) for h in head_stats])
    maxs = np.stack([np.asarray(h["actions"]["max"], np.float64) for h in head_stats])
    lo = np.nanmin(np.where(np.isfinite(mins), mins, np.nan), axis=0)
    hi = np.nanmax(np.where(np.isfinite(maxs), maxs, np.nan), axis=0)
    z = np.zeros_like(lo)
    return {"actions": {"min": lo.astype(np.float32), "max": hi.astype(np.float32), "mean": z.astype(np.float32),
                        "std": z.astype(np.float32) + 1}}


def fit(chunks: np.ndarray, vocab_size: int = 2048, scale: float = 10.0, holdout: float = 0.1,
        max_token_length: int | None = None, seed: int = 0) -> tuple[BpeDctActionTokenizer, dict]:
    """Learns the merge table on all but a held-out share of already NORMALISED chunks ``(N, T, D)`` and checks the
    round trip on the rest.  Returns the tokenizer and the report block."""
    order = np.random.default_rng(seed).permutation(len(chunks))
    n_hold = min(max(1, int(len(chunks) * holdout)), 4096) if len(chunks) > 1 else 0
    held, train = chunks[order[:n_hold]], chunks[order[n_hold:]] if n_hold else chunks
    t0 = time.perf_counter()
    tok = BpeDctActionTokenizer(scale=scale).fit(train, vocab_size=vocab_size)
    fit_s = time.perf_counter() - t0
    check = held if n_hold else train[:256]
    ids = tok(check)
    rec = tok.decode(ids)
    lengths = np.asarray([len(x) for x in ids])
    report = {"chunks": int(len(chunks)), "held_out": int(len(check)), "vocab_size": tok.vocab_size,
              "base_symbols": tok.base, "merges": len(tok.merges), "fit_seconds": fit_s,
              "tokens_per_chunk_mean": float(lengths.mean()),
              "tokens_per_chunk_percentiles": {f"p{q}": float(np.percentile(lengths, q)) for q in (50, 90, 99, 100)},
              "symbols_per_chunk_mean": float(np.mean([len(x) for x in tok._symbols(check)])),
              "reconstruction_rmse": float(np.sqrt(np.mean((rec - check) ** 2))),
              "reconstruction_max_abs": float(np.abs(rec - check).max())}
    if max_token_length is not None:
        report["share_above_max_token_length"] = float((lengths > max_token_length).mean())
    if len(tok.merges) < MIN_MERGE_HEADROOM:
        logging.warning("only %d merges were learned (vocabulary %d, base alphabet %d): the table barely compresses; "
                        "raise --vocab-size or fit on more chunks", len(tok.merges), vocab_size, tok.base)
    return tok, report


def save(tok: BpeDctActionTokenizer, out_dir: Path, config_version: int) -> None:
    """The tokenizer and, beside it, the convention its corpus was normalised under: a policy that resolves to the
    other convention refuses the tokenizer at load time instead of tokenizing values the corpus never saw."""
    out_dir.mkdir(parents=True, exist_ok=True)
    tok.save(out_dir / TOKENIZER_FILE)
    (out_dir / ACTION_NORM_META_FILE).write_text(json.dumps(
        {"config_version": int(config_version), "zero_range_center": bool(config_version >= 1)}, indent=2))


def run(args: argparse.Namespace) -> dict[str, Any]:
    from ..datasets.factory import make_dataset_mixture
    out_dir = args.out_dir / "pilot" if args.pilot else args.out_dir
    total = min(args.total_chunks, PILOT_CHUNKS) if args.pilot else args.total_chunks
    if total != args.total_chunks:
        logging.info("pilot: --total-chunks lowered from %d to %d", args.total_chunks, total)
    out_dir.mkdir(parents=True, exist_ok=True)
    logging.info("fitting under config_version=%d (zero-range dims map to %s, eps %g)", args.config_version,
                 "0" if args.config_version >= 1 else "-1", OPENPI_EPS if args.config_version >= 1 else LEGACY_EPS)
    mixture_cfg, digest = parse_mixture(args.mixture_json)
    logging.info("mixture: %d dataset(s), hash %s, action_freq %s", len(mixture_cfg.datasets), digest[:12],
                 "per dataset (native fps)" if mixture_cfg.action_freq is None else f"{mixture_cfg.action_freq:g}")
    t0 = time.perf_counter()
    cfg = build_train_cfg(mixture_cfg, chunk_size=args.chunk_size, action_dim=args.action_dim,
                          max_state_dim=args.max_state_dim, seed=args.seed)
    built = make_dataset_mixture(cfg)
    mix = built[0] if isinstance(built, tuple) else built
    build_s = time.perf_counter() - t0
    meta = mix.meta
    budgets = compute_budgets(list(mix.weights), total)
    rng = np.random.default_rng(args.seed)
    t0 = time.perf_counter()
    parts, heads, per_dataset, errors = [], [], [], {}
    widest = 0
    for i, (tagged, name, n) in enumerate(zip(mix.datasets, mix.names, budgets)):
        ds = getattr(tagged, "dataset", tagged)
        if n == 0 or getattr(ds, "is_vqa", False) or not hasattr(ds, "_numeric"):
            per_dataset.append(0)          # question-answer and synthetic members carry no action columns
            continue
        try:
            raw = sample_dataset_chunks(ds, n, args.chunk_size, mixture_cfg.action_freq, rng)
        except Exception as exc:  # noqa: BLE001 - one unreadable member is reported, the fit goes on with the rest
            logging.warning("dataset %s: no chunks sampled (%r)", name, exc)
            errors[i] = repr(exc)
            per_dataset.append(0)
            continue
        widest = max(widest, raw.shape[2])
        parts.append(pad_to_action_dim(raw, args.action_dim))
        heads.append(np.full(len(raw), meta.dataset_to_norm_index[name], np.int64))
        per_dataset.append(int(len(raw)))
    if not parts:
        raise RuntimeError("no chunks sampled: see the warnings above")
    if widest > args.action_dim:
        logging.warning("action dims %d.. of the widest dataset (%d) are cut: the policy never sees them", args.action_dim, widest)
    chunks, head_index = np.concatenate(parts), np.concatenate(heads)
    head_stats = [{"actions": h["actions"]} for h in meta.per_norm_key_stats]
    if not args.per_head_norm:
        head_stats, head_index = [pooled_head(head_stats)], np.zeros_like(head_index)
    normalised = normalize_chunks(chunks, head_index, head_stats, config_version=args.config_version,
                                  action_dim=args.action_dim)
    sample_s = time.perf_counter() - t0
    report: dict[str, Any] = {
        "mixture_json": str(args.mixture_json), "mixture_hash_sha256": digest, "n_datasets": len(mixture_cfg.datasets),
        "action_freq": mixture_cfg.action_freq, "chunk_size": args.chunk_size, "action_dim": args.action_dim,
        "config_version": args.config_version, "zero_range_center": args.config_version >= 1,
        "vocab_size": args.vocab_size, "scale": args.scale, "max_token_length": args.max_token_length,
        "seed": args.seed, "total_chunks_target": total, "total_chunks_actual": int(len(normalised)),
        "sampler": "numeric_columns", "normalization": "per_robot_type_control_mode" if args.per_head_norm else "global",
        "dataset_names": list(mix.names), "per_dataset_chunks": per_dataset, "sample_errors": errors,
        "per_dataset_norm_keys": [meta.norm_keys[meta.dataset_to_norm_index[n]] for n in mix.names],
        "n_norm_heads": len(meta.norm_keys),
        "per_head_action_stats": {k: {"min": np.asarray(s["actions"]["min"]).tolist(),
                                      "max": np.asarray(s["actions"]["max"]).tolist()}
                                  for k, s in zip(meta.norm_keys, meta.per_norm_key_stats)},
        "delta_action_state_map": meta.delta_action_state_map,
        "normalised_range": [float(normalised.min()), float(normalised.max())],
        "timings_seconds": {"build_mixture": build_s, "sample_and_normalise": sample_s},
        "pilot": bool(args.pilot),
    }
    if not args.skip_fit:
        tok, fit_report = fit(normalised, args.vocab_size, args.scale, args.holdout, args.max_token_length, args.seed)
        save(tok, out_dir, args.config_version)
        report["roundtrip"] = fit_report
        report["timings_seconds"]["fit"] = fit_report["fit_seconds"]
    (out_dir / REPORT_FILE).write_text(json.dumps(report, indent=2, default=str))
    logging.info("report written to %s", out_dir / REPORT_FILE)
    return report


def main(argv: list[str] | None = None) -> int:
    args = parse_args(argv)
    logging.basicConfig(level=getattr(logging, str(args.log_level).upper(), logging.INFO),
                        format="%(asctime)s %(levelname)s %(message)s")
    report = run(args)
    print(json.dumps({k: report[k] for k in ("total_chunks_actual", "n_norm_heads", "normalization") if k in report}
                     | ({"roundtrip": report["roundtrip"]} if "roundtrip" in report else {}), indent=2))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
