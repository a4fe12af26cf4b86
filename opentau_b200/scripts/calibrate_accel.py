"""``opentau-accel-calibrate``: fit the CUSUM failure detector from recorded rollouts
(reference ``src/opentau/scripts/calibrate_accel.py``).

Input: a JSON / JSONL file of episodes ``{"accel": [z_0, z_1, ...], "success": bool}`` (what ``opentau-eval`` and the
gRPC server log when ``accel_prefix`` is set).  Successful episodes are split into a calibration part and a held-out
part; the fitted threshold is written next to the checkpoint and scored on the held-out successes plus all failures.

    opentau-accel-calibrate --episodes rollouts.jsonl --out checkpoints/last --alpha 0.1
"""

from __future__ import annotations

import argparse
import json
import logging
from pathlib import Path

import numpy as np

from ..utils.accel_detector import DEFAULT_ALPHA, DEFAULT_SLACK_C, calibrate, evaluate


def load_episodes(path: str | Path) -> tuple[list[list[float]], list[bool]]:
    text = Path(path).read_text().strip()
    rows = json.loads(text) if text.startswith("[") else [json.loads(line) for line in text.splitlines() if line.strip()]
    return [list(map(float, r["accel"])) for r in rows], [bool(r["success"]) for r in rows]


def main(argv: list[str] | None = None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--episodes", required=True)
    ap.add_argument("--out", required=True, help="directory (or file) for the calibration JSON")
    ap.add_argument("--alpha", type=float, default=DEFAULT_ALPHA)
    ap.add_argument("--slack-c", type=float, default=DEFAULT_SLACK_C)
    ap.add_argument("--holdout", type=float, default=0.3, help="fraction of successful episodes kept for scoring")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    eps, ok = load_episodes(a.episodes)
    good = [e for e, s in zip(eps, ok) if s]
    bad = [e for e, s in zip(eps, ok) if not s]
    perm = np.random.default_rng(a.seed).permutation(len(good))
    n_hold = int(len(good) * a.holdout)
    held = [good[i] for i in perm[:n_hold]]
    fit = [good[i] for i in perm[n_hold:]]
    cal = calibrate(fit, alpha=a.alpha, slack_c=a.slack_c)
    where = cal.save(a.out)
    report = evaluate(held + bad, [True] * len(held) + [False] * len(bad), cal)
    logging.info("calibration written to %s: mu0=%.4g sigma=%.4g eta=%.4g (M=%d)", where, cal.mu0, cal.sigma, cal.eta,
                 cal.num_calibration_episodes)
    print(json.dumps({"calibration": cal.to_dict(), "held_out": report}, indent=2))
    return {"calibration": cal, "report": report}


if __name__ == "__main__":
    main()
