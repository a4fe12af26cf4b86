"""Fit the discrete action tokenizer (DCT + byte-pair merges) on the action chunks of a dataset mixture
(reference ``src/opentau/scripts/fit_fast_tokenizer.py``).

Chunks are normalised to [-1, 1] with the 1st / 99th percentiles of each action dimension (robust min-max); the
percentiles are written next to the tokenizer as ``opentau_action_norm.json`` so that training and serving normalise
identically.  Reports compression (tokens per chunk) and reconstruction error on a held-out part.

    python -m opentau_b200.scripts.fit_fast_tokenizer --config_path=cfg.json --output tok_dir --vocab-size 2048
"""

from __future__ import annotations

import argparse
import json
import logging
from pathlib import Path

import numpy as np

from ..configs import parser
from ..configs.train import TrainPipelineConfig
from ..utils.tokenizer import BpeDctActionTokenizer

NORM_SIDECAR = "opentau_action_norm.json"
TOKENIZER_FILE = "action_tokenizer.json"


def collect_chunks(mixture, max_chunks: int, seed: int = 0) -> np.ndarray:
    rng = np.random.default_rng(seed)
    idx = rng.choice(len(mixture), size=min(max_chunks, len(mixture)), replace=False)
    out = []
    for i in idx:
        it = mixture.get_global(int(i))
        if bool(it["action_is_pad"].all()):
            continue
        d = int(it["real_action_dim"])
        out.append(it["actions"].float().numpy()[:, :d])
    width = max(c.shape[1] for c in out)
    return np.stack([np.pad(c, ((0, 0), (0, width - c.shape[1]))) for c in out])


def fit(chunks: np.ndarray, vocab_size: int = 2048, scale: float = 10.0, holdout: float = 0.1) -> tuple[BpeDctActionTokenizer, dict, dict]:
    lo, hi = np.quantile(chunks, 0.01, axis=(0, 1)), np.quantile(chunks, 0.99, axis=(0, 1))
    span = np.where(hi - lo < 1e-8, 1.0, hi - lo)
    norm = np.clip((chunks - lo) / span * 2 - 1, -1.5, 1.5)
    n_hold = max(1, int(len(norm) * holdout))
    tok = BpeDctActionTokenizer(scale=scale).fit(norm[n_hold:], vocab_size=vocab_size)
    held = norm[:n_hold]
    ids = tok(held)
    rec = tok.decode(ids)
    report = {"chunks": int(len(norm)), "vocab_size": tok.vocab_size, "merges": len(tok.merges),
              "tokens_per_chunk_mean": float(np.mean([len(x) for x in ids])),
              "symbols_per_chunk_mean": float(np.mean([len(x) for x in tok._symbols(held)])),
              "reconstruction_rmse": float(np.sqrt(np.mean((rec - held) ** 2)))}
    return tok, {"q01": lo.tolist(), "q99": hi.tolist()}, report


def main() -> None:
    from ..datasets.factory import make_dataset_mixture
    from ..utils.logging_utils import init_logging
    init_logging()
    ap = argparse.ArgumentParser(add_help=False)
    ap.add_argument("--output", required=True)
    ap.add_argument("--vocab-size", type=int, default=2048)
    ap.add_argument("--max-chunks", type=int, default=20000)
    ap.add_argument("--scale", type=float, default=10.0)
    a, rest = ap.parse_known_args()
    cfg: TrainPipelineConfig = parser.parse_config(TrainPipelineConfig, rest)
    res = make_dataset_mixture(cfg)
    mix = res[0] if isinstance(res, tuple) else res
    tok, norm, report = fit(collect_chunks(mix, a.max_chunks, cfg.seed or 0), a.vocab_size, a.scale)
    out = Path(a.output)
    tok.save(out / TOKENIZER_FILE)
    (out / NORM_SIDECAR).write_text(json.dumps(norm))
    logging.info("tokenizer written to %s: %s", out, report)
    print(json.dumps(report, indent=2))


if __name__ == "__main__":
    main()
