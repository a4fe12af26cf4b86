"""``opentau-accel-calibrate``: fit the CUSUM failure-detection threshold from recorded ``accel`` streams
(reference ``src/opentau/scripts/calibrate_accel.py:71-293``).

The score is free; the detector is not, and this is where its cost is paid: offline, once.  Only SUCCESSFUL rollouts
are needed (no failure labels).  The real cost is the number of episodes: the threshold is an order statistic of
per-episode CUSUM peaks, so ``alpha = 0.1`` needs at least 9 successes (50 is a comfortable operating point).

Input, either of
  * the ``eval_info.json`` of an evaluation run with accel armed (``OPENTAU_ACCEL_PREFIX=auto opentau-eval ...``):
    per task, ``accel[task].streams`` is index-aligned with ``per_episode[task]``;
  * a JSON / JSONL list of episodes ``{"accel": [z_0, z_1, ...], "success": bool[, "task": name]}`` (what a serving
    log can be turned into).

    opentau-accel-calibrate outputs/eval/eval_info.json --alpha 0.1 --out outputs/accel [--per-task] [--holdout 0.3]

``--per-task`` fits one threshold per task rather than one pooled threshold: task difficulty shifts the score's
location, and a pooled threshold under-detects on the hard tasks.  Without ``--holdout`` the printed rates are
measured on the episodes the threshold was fitted from and are optimistic; the conformal guarantee is on the
out-of-sample false-alarm rate.  With ``--holdout F`` that fraction of the successful episodes is kept out of the fit
and scored together with all failures.
"""

from __future__ import annotations

import argparse
import json
import logging
import math
from dataclasses import replace
from pathlib import Path

import numpy as np

from ..policies.accel import AccelProvenance
from ..utils.accel_detector import DEFAULT_ALPHA, DEFAULT_SLACK_C, calibrate, conformal_rank, evaluate

logger = logging.getLogger(__name__)


def load_tasks(path: str | Path) -> list[dict]:
    """-> ``[{"task": name, "accels": [[...], ...], "successes": [...], "provenance": dict | None}]``.  A task whose
    stream and outcome lists differ in length is dropped rather than paired up: a stream labelled with another
    episode's outcome would poison the calibration invisibly."""
    path = Path(path)
    if path.is_dir():
        path = path / "eval_info.json"
    if not path.exists():
        raise FileNotFoundError(f"No eval_info.json or episode file at {path}.")
    text = path.read_text().strip()
    try:
        payload = json.loads(text)
    except json.JSONDecodeError:                 # one JSON object per line
        payload = [json.loads(line) for line in text.splitlines() if line.strip()]
    tasks: list[dict] = []
    if isinstance(payload, dict) and "per_episode" in payload:
        accel = payload.get("accel") or {}
        for name, episodes in payload["per_episode"].items():
            rec = accel.get(name)
            if not rec or not rec.get("streams"):
                continue
            tasks.append({"task": name, "accels": rec["streams"], "successes": [bool(e["success"]) for e in episodes],
                          "provenance": rec.get("provenance")})
    else:
        rows = payload if isinstance(payload, list) else [payload]
        by_task: dict[str, dict] = {}
        for r in rows:
            t = by_task.setdefault(str(r.get("task", "all")), {"task": str(r.get("task", "all")), "accels": [],
                                                               "successes": [], "provenance": r.get("provenance")})
            t["accels"].append([float(z) for z in r["accel"]])
            t["successes"].append(bool(r["success"]))
        tasks = list(by_task.values())
    kept = []
    for t in tasks:
        if len(t["accels"]) != len(t["successes"]):
            logger.warning("%s: %d accel stream(s) for %d success flag(s); skipping this task rather than pairing a "
                           "stream with the wrong episode", t["task"], len(t["accels"]), len(t["successes"]))
            continue
        kept.append(t)
    return kept


def resolve_provenance(tasks: list[dict]) -> AccelProvenance | None:
    """The provenance shared by ``tasks`` (compared on the distribution-shifting fields only; the per-sample fields
    are cleared), or ``None`` when none was recorded or the tasks disagree -- an unlabelled calibration skips the
    comparability check at apply time instead of passing it on false pretences."""
    provs = [AccelProvenance.from_dict(t["provenance"]) for t in tasks if t.get("provenance")]
    seen = {json.dumps({f: getattr(p, f) for f in AccelProvenance.COMPARABLE_FIELDS}, sort_keys=True) for p in provs}
    if not seen:
        logger.warning("no task recorded an accel provenance; the calibration will be unlabelled")
        return None
    if len(seen) > 1:
        logger.warning("tasks disagree on accel provenance (%d distinct); the calibration is left unlabelled -- fit "
                       "per task instead", len(seen))
        return None
    return replace(provs[0], dataset_index=(), num_scored_dims=())


def fit(tasks: list[dict], *, alpha: float, slack_c: float, label: str, holdout: float = 0.0, seed: int = 0) -> dict | None:
    """One calibration over the pooled ``tasks`` and its evaluation; ``None`` when there are too few successful
    episodes to certify ``alpha``."""
    good = [s for t in tasks for s, ok in zip(t["accels"], t["successes"]) if ok and len(s)]
    bad = [s for t in tasks for s, ok in zip(t["accels"], t["successes"]) if not ok and len(s)]
    if not good:
        logger.warning("%s: no successful episodes with an accel stream; skipping", label)
        return None
    held: list = []
    if holdout > 0.0:
        perm = np.random.default_rng(seed).permutation(len(good))
        n_hold = int(len(good) * holdout)
        held, good = [good[i] for i in perm[:n_hold]], [good[i] for i in perm[n_hold:]]
    try:
        rank = conformal_rank(len(good), alpha)
    except ValueError as exc:
        logger.warning("%s: %s", label, exc)
        return None
    cal = calibrate(good, alpha=alpha, slack_c=slack_c, provenance=resolve_provenance(tasks))
    scored, flags = ((held + bad, [True] * len(held) + [False] * len(bad)) if holdout > 0.0
                     else (good + bad, [True] * len(good) + [False] * len(bad)))
    metrics = evaluate(scored, flags, cal)
    logger.info("%s: fitted on %d successful episode(s) (order statistic %d), eta=%.6g; %s TPR=%.3f false-alarm=%.3f "
                "median lead=%.1f chunks over %d failing / %d successful", label, len(good), rank, cal.eta,
                "held-out" if holdout > 0.0 else "held-in", metrics["true_positive_rate"], metrics["false_alarm_rate"],
                metrics["median_lead"], int(metrics["n_failed"]), int(metrics["n_successful"]))
    return {"calibration": cal, "metrics": metrics, "num_successful": len(good), "held_out": holdout > 0.0}


def main(argv: list[str] | None = None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("eval_info", nargs="?", help="eval_info.json (or its directory), or a JSON / JSONL episode list")
    ap.add_argument("--episodes", help="same as the positional argument")
    ap.add_argument("--alpha", type=float, default=DEFAULT_ALPHA, help="target false-alarm rate")
    ap.add_argument("--slack-c", type=float, default=DEFAULT_SLACK_C, help="CUSUM slack, in sigmas")
    ap.add_argument("--out", default="outputs/accel", help="output directory")
    ap.add_argument("--per-task", action="store_true", help="one threshold per task instead of one pooled threshold")
    ap.add_argument("--holdout", type=float, default=0.0, help="fraction of successful episodes kept out for scoring")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    source = a.eval_info or a.episodes
    if not source:
        ap.error("give an eval_info.json or an episode file")
    tasks = load_tasks(source)
    if not tasks:
        raise SystemExit(f"No task in {source} recorded accel streams. Re-run the evaluation with "
                         "OPENTAU_ACCEL_PREFIX=auto (or policy.accel_prefix set).")
    out = Path(a.out)
    out.mkdir(parents=True, exist_ok=True)
    groups = [(t["task"].replace("/", "__"), [t]) for t in tasks] if a.per_task else [("pooled", tasks)]
    summary: dict[str, dict] = {}
    results: dict[str, dict] = {}
    for label, members in groups:
        res = fit(members, alpha=a.alpha, slack_c=a.slack_c, label=label, holdout=a.holdout, seed=a.seed)
        if res is None:
            continue
        path = res["calibration"].save(out / f"accel_calibration__{label}.json")
        results[label] = res
        summary[label] = {"path": str(path), "num_successful": res["num_successful"], "eta": res["calibration"].eta,
                          "held_out": res["held_out"], **res["metrics"]}
    if not summary:
        raise SystemExit(f"No calibration could be fitted at alpha={a.alpha}: every group had fewer than the "
                         f"{math.ceil(1.0 / a.alpha) - 1} successful episodes a finite split-conformal threshold needs "
                         "at that rate. Collect more successful rollouts, drop --per-task to pool them, or raise --alpha.")
    (out / "accel_calibration_summary.json").write_text(json.dumps(summary, indent=2) + "\n")
    if a.holdout <= 0.0:
        logger.warning("the rates above are measured on the SAME episodes the threshold was fitted from and are "
                       "optimistic; measure the true-positive rate on a disjoint set of rollouts (or use --holdout)")
    print(json.dumps(summary, indent=2))
    first = next(iter(results.values()))
    return {"calibration": first["calibration"], "report": first["metrics"], "summary": summary, "results": results}


if __name__ == "__main__":
    logging.basicConfig(level=logging.INFO)
    main()
