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


def test_calibration_from_eval_info_pooled_and_per_task(tmp_path):
    """The evaluator's own output feeds the tool: per-task streams index-aligned with per-episode outcomes, one
    provenance for the pool (per-sample fields cleared), per-task files on request, and a clear refusal when no
    group has enough successful episodes for the requested rate."""
    rng = np.random.default_rng(1)
    prov = {"policy_type": "pi05", "num_steps": 10, "prefix": 9, "chunk_size": 50, "n_action_steps": 50, "max_delay": 0,
            "action_norm_mode": "MEAN_STD", "has_delta_action_map": False, "velocity_dtype": "bfloat16",
            "num_scored_dims": [7], "dataset_index": [0], "n_candidates": 1}

    def task(n_ok, n_bad):
        streams = [list(rng.normal(1.0, 0.1, size=30)) for _ in range(n_ok)]
        streams += [list(rng.normal(1.0, 0.1, size=15)) + list(rng.normal(1.6, 0.1, size=15)) for _ in range(n_bad)]
        eps = [{"episode_ix": i, "success": i < n_ok} for i in range(n_ok + n_bad)]
        return streams, eps
    s_a, e_a = task(30, 6)
    s_b, e_b = task(12, 3)
    info = {"per_episode": {"g/0": e_a, "g/1": e_b, "g/2": [{"success": True}]},
            "accel": {"g/0": {"streams": s_a, "provenance": prov},
                      "g/1": {"streams": s_b, "provenance": {**prov, "dataset_index": [1], "num_scored_dims": [6]}}}}
    (tmp_path / "eval_info.json").write_text(json.dumps(info))
    out = calibrate_main([str(tmp_path), "--out", str(tmp_path / "cal"), "--alpha", "0.1"])
    cal = out["calibration"]
    assert set(out["summary"]) == {"pooled"} and out["summary"]["pooled"]["num_successful"] == 42
    assert out["report"]["true_positive_rate"] == 1.0 and cal.provenance.prefix == 9
    assert cal.provenance.dataset_index == () and cal.provenance.num_scored_dims == ()
    assert CusumCalibration.load(tmp_path / "cal" / "accel_calibration__pooled.json") == cal
    per = calibrate_main([str(tmp_path / "eval_info.json"), "--out", str(tmp_path / "per"), "--per-task", "--holdout", "0.2"])
    assert set(per["summary"]) == {"g__0", "g__1"} and per["summary"]["g__0"]["held_out"] is True
    assert (tmp_path / "per" / "accel_calibration_summary.json").exists()
    with pytest.raises(SystemExit, match="No calibration could be fitted"):
        calibrate_main([str(tmp_path), "--out", str(tmp_path / "x"), "--alpha", "0.01"])
    info["accel"]["g/1"]["provenance"] = {**prov, "prefix": 4}
    (tmp_path / "eval_info.json").write_text(json.dumps(info))
    mixed = calibrate_main([str(tmp_path), "--out", str(tmp_path / "m")])
    assert mixed["calibration"].provenance is None            # disagreeing tasks leave the pool unlabelled
