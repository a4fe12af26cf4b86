"""CUSUM / split-conformal failure detector and its calibration CLI."""

import json

import numpy as np
import pytest

from opentau_b200.scripts.calibrate_accel import main as calibrate_main
from opentau_b200.utils.accel_detector import (CusumCalibration, calibrate, conformal_rank, cusum_stream, detect,
                                               evaluate)


def test_cusum_recursion_and_nan_handling():
    s = cusum_stream([1.0, 3.0, float("nan"), 0.0, 5.0], mu0=1.0, k=0.5)
    assert np.allclose(s, [0.0, 1.5, 1.5, 0.0, 3.5])


def test_conformal_rank_matches_the_paper_and_rejects_small_samples():
    assert conformal_rank(50, 0.1) == 46
    with pytest.raises(ValueError, match="at least 9"):
        conformal_rank(5, 0.1)


def test_detector_flags_drifting_episodes_and_keeps_false_alarms_near_alpha(tmp_path):
    rng = np.random.default_rng(0)
    good = [list(rng.normal(1.0, 0.1, size=int(rng.integers(25, 50)))) for _ in range(80)]
    bad = []
    for _ in range(20):
        ep = list(rng.normal(1.0, 0.1, size=40))
        ep[20:] = list(np.asarray(ep[20:]) + 0.5)           # persistent drift from chunk 20 on
        bad.append(ep)
    cal = calibrate(good[:50], alpha=0.1)
    rep = evaluate(good[50:] + bad, [True] * 30 + [False] * 20, cal)
    assert rep["true_positive_rate"] == 1.0 and rep["false_alarm_rate"] <= 0.3 and rep["median_lead"] >= 15
    r = detect(bad[0], cal)
    assert r.alarmed and 20 <= r.alarm_index <= 24 and r.lead == 39 - r.alarm_index
    cal2 = CusumCalibration.load(cal.save(tmp_path))
    assert cal2 == cal
    rows = [{"accel": e, "success": True} for e in good] + [{"accel": e, "success": False} for e in bad]
    (tmp_path / "eps.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    out = calibrate_main(["--episodes", str(tmp_path / "eps.jsonl"), "--out", str(tmp_path), "--alpha", "0.1"])
    assert out["report"]["true_positive_rate"] == 1.0
