"""Failure detector over the per-chunk ``accel`` stream: one-sided CUSUM with a split-conformal threshold
(reference ``src/opentau/utils/accel_detector.py:82-403``).

``S_0 = 0,  S_t = max(0, S_{t-1} + z_t - mu0 - k)`` with slack ``k = c * sigma``; the alarm fires at the first ``t``
with ``S_t > eta``.  ``mu0`` / ``sigma`` come from the pooled chunk scores of held-out SUCCESSFUL rollouts; ``eta``
is an order statistic of the per-EPISODE peaks (the exchangeable unit is the episode — chunk scores inside one
episode are strongly dependent), rank ``ceil((M + 1)(1 - alpha))``.  Non-finite scores carry ``S`` forward.
Nothing here runs in the serving hot path.
"""

from __future__ import annotations

import json
import logging
import math
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Sequence

import numpy as np

from ..policies.accel import AccelProvenance, assert_comparable

DEFAULT_SLACK_C = 0.25
DEFAULT_ALPHA = 0.1
CALIBRATION_FILENAME = "opentau_accel_calibration.json"


def cusum_stream(scores: Sequence[float], *, mu0: float, k: float) -> np.ndarray:
    out = np.empty(len(scores), dtype=np.float64)
    s = 0.0
    for i, z in enumerate(scores):
        if math.isfinite(z):
            s = max(0.0, s + float(z) - mu0 - k)
        out[i] = s
    return out


def episode_peak(scores: Sequence[float], *, mu0: float, k: float) -> float:
    return 0.0 if len(scores) == 0 else float(cusum_stream(scores, mu0=mu0, k=k).max())


def conformal_rank(num_calibration: int, alpha: float) -> int:
    if not 0.0 < alpha < 1.0:
        raise ValueError(f"alpha must be in (0, 1), got {alpha}.")
    rank = math.ceil((num_calibration + 1) * (1.0 - alpha))
    if rank > num_calibration:
        raise ValueError(f"alpha={alpha} needs at least {math.ceil(1.0 / alpha) - 1} calibration episodes for a finite "
                         f"split-conformal threshold, got {num_calibration}. Collect more successful rollouts or raise alpha.")
    return rank


@dataclass(frozen=True)
class CusumCalibration:
    mu0: float
    sigma: float
    slack_c: float
    eta: float
    alpha: float
    num_calibration_episodes: int
    num_calibration_chunks: int
    provenance: AccelProvenance | None = None

    @property
    def k(self) -> float:
        return self.slack_c * self.sigma

    def to_dict(self) -> dict:
        d = asdict(self)
        d["provenance"] = asdict(self.provenance) if self.provenance is not None else None
        return d

    @classmethod
    def from_dict(cls, payload: dict) -> "CusumCalibration":
        p = dict(payload)
        prov = p.pop("provenance", None)
        return cls(**p, provenance=AccelProvenance.from_dict(prov) if prov else None)

    def save(self, path: str | Path) -> Path:
        path = Path(path)
        if path.is_dir():
            path = path / CALIBRATION_FILENAME
        path.write_text(json.dumps(self.to_dict(), indent=2))
        return path

    @classmethod
    def load(cls, path: str | Path) -> "CusumCalibration":
        path = Path(path)
        if path.is_dir():
            path = path / CALIBRATION_FILENAME
        return cls.from_dict(json.loads(path.read_text()))


def calibrate(episodes: Sequence[Sequence[float]], *, alpha: float = DEFAULT_ALPHA, slack_c: float = DEFAULT_SLACK_C,
              provenance: AccelProvenance | None = None) -> CusumCalibration:
    """Fits ``mu0, sigma, eta`` on the accel streams of successful rollouts."""
    episodes = [[z for z in ep] for ep in episodes if len(ep)]
    if not episodes:
        raise ValueError("no calibration episodes")
    pooled = np.asarray([z for ep in episodes for z in ep if math.isfinite(z)], dtype=np.float64)
    if pooled.size == 0:
        raise ValueError("calibration episodes hold no finite score")
    mu0, sigma = float(pooled.mean()), float(pooled.std())
    if sigma == 0.0:
        logging.warning("accel calibration scale is exactly zero (%d pooled chunks): any increase will alarm", pooled.size)
    k = slack_c * sigma
    peaks = np.sort([episode_peak(ep, mu0=mu0, k=k) for ep in episodes])
    eta = float(peaks[conformal_rank(len(episodes), alpha) - 1])
    return CusumCalibration(mu0, sigma, slack_c, eta, alpha, len(episodes), int(pooled.size), provenance)


@dataclass(frozen=True)
class DetectionResult:
    alarm_index: int | None
    lead: int | None
    peak: float
    statistic: np.ndarray

    @property
    def alarmed(self) -> bool:
        return self.alarm_index is not None


def detect(scores: Sequence[float], calibration: CusumCalibration, *, provenance: AccelProvenance | None = None) -> DetectionResult:
    if provenance is not None and calibration.provenance is not None:
        assert_comparable(calibration.provenance, provenance)
    st = cusum_stream(scores, mu0=calibration.mu0, k=calibration.k)
    above = np.flatnonzero(st > calibration.eta)
    idx = int(above[0]) if above.size else None
    return DetectionResult(idx, (len(scores) - 1 - idx) if idx is not None else None, float(st.max()) if st.size else 0.0, st)


def evaluate(episodes: Sequence[Sequence[float]], successes: Sequence[bool], calibration: CusumCalibration) -> dict[str, float]:
    if len(episodes) != len(successes):
        raise ValueError(f"episodes ({len(episodes)}) and successes ({len(successes)}) differ in length.")
    res = [detect(ep, calibration) for ep in episodes]
    failed = [r for r, ok in zip(res, successes) if not ok]
    passed = [r for r, ok in zip(res, successes) if ok]
    leads = [r.lead for r in failed if r.alarmed]
    return {"true_positive_rate": float(np.mean([r.alarmed for r in failed])) if failed else float("nan"),
            "false_alarm_rate": float(np.mean([r.alarmed for r in passed])) if passed else float("nan"),
            "median_lead": float(np.median(leads)) if leads else float("nan"),
            "n_failed": float(len(failed)), "n_successful": float(len(passed))}
