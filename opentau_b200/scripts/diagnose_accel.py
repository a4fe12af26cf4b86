"""``opentau-accel-diagnose``: measure what the ``accel`` score of a checkpoint is made of -- run this before any
threshold is calibrated (reference ``src/opentau/scripts/diagnose_accel.py:119-1041``).

The numerator of ``accel`` is a difference of nearly equal velocity vectors, and policies are served in bf16, so a
positive rounding floor sits beneath every score and compresses the "certain" end of the range.  On the checkpoint
itself, changing nothing in it, this tool measures

1. the dtype floor: each observation denoised with the SAME pinned noise in fp32 and in the serving dtype; the field,
   the conditioning and the draw are identical, so the difference is rounding alone;
2. the stochasticity: one observation, noise redrawn each time (what a detector's calibration has to absorb);
3. the prefix sweep: mean ``accel_p`` for every ``p`` from one pass at the full schedule.  Descriptive only: both sums
   grow with ``p``, so the largest value says nothing about the best prefix;
4. the prefix study: ``K`` independent denoises per observation give the posterior spread of the action chunk (the
   quantity ``accel`` is meant to track); the figure of merit for a prefix is the rank correlation, across
   observations, between ``accel_p`` and that spread.

The go / no-go: is the spread of the score between observations large against the dtype floor?  If it is not, a
threshold on this checkpoint measures arithmetic.

    opentau-accel-diagnose --config_path=<checkpoint or config> [--policy.device=cuda]

Cost knobs (environment, because the pipeline config has no fields for them): ``OPENTAU_ACCEL_OBSERVATIONS`` (24),
``OPENTAU_ACCEL_RESAMPLES`` (K, 32; 0 skips the study), ``OPENTAU_ACCEL_MEASURE_DTYPE_FLOOR`` (1; 0 skips the fp32 leg,
which holds a second, wider copy of the weights).
"""

from __future__ import annotations

import json
import logging
import math
import os
from dataclasses import dataclass, field
from pathlib import Path

import torch

from ..configs import parser
from ..configs.train import TrainPipelineConfig
from ..policies.accel import action_dim_scale, default_prefix, record_traces, resolve_action_dim_mask
from ..policies.factory import make_policy
from ..policies.utils import to_dtype_preserving_siglip_float32
from ..utils.utils import init_logging

logger = logging.getLogger(__name__)

RESAMPLES_ENV = "OPENTAU_ACCEL_RESAMPLES"
OBSERVATIONS_ENV = "OPENTAU_ACCEL_OBSERVATIONS"
DTYPE_FLOOR_ENV = "OPENTAU_ACCEL_MEASURE_DTYPE_FLOOR"


def _finite(values) -> list[float]:
    return [float(v) for v in values if math.isfinite(v)]


def _mean(values) -> float:
    f = _finite(values)
    return sum(f) / len(f) if f else float("nan")


def _std(values) -> float:
    f = _finite(values)
    if not f:
        return float("nan")
    m = sum(f) / len(f)
    return math.sqrt(sum((v - m) ** 2 for v in f) / len(f))


def _median(values) -> float:
    f = sorted(_finite(values))
    if not f:
        return float("nan")
    h = len(f) // 2
    return f[h] if len(f) % 2 else 0.5 * (f[h - 1] + f[h])


def _ranks(xs: list[float]) -> list[float]:
    """Average ranks (ties share the mean of their positions)."""
    order = sorted(range(len(xs)), key=lambda i: xs[i])
    out = [0.0] * len(xs)
    i = 0
    while i < len(order):
        j = i
        while j + 1 < len(order) and xs[order[j + 1]] == xs[order[i]]:
            j += 1
        for k in range(i, j + 1):
            out[order[k]] = 0.5 * (i + j) + 1.0
        i = j + 1
    return out


def spearman(xs: list[float], ys: list[float]) -> float:
    """Rank correlation with non-finite pairs dropped; NaN with fewer than three pairs or a constant side.  Rank
    based on purpose: the relation between ``accel_p`` and the spread is monotone at best, not linear."""
    pairs = [(x, y) for x, y in zip(xs, ys) if math.isfinite(x) and math.isfinite(y)]
    if len(pairs) < 3:
        return float("nan")
    rx, ry = _ranks([p[0] for p in pairs]), _ranks([p[1] for p in pairs])
    mx, my = sum(rx) / len(rx), sum(ry) / len(ry)
    sxx = sum((a - mx) ** 2 for a in rx)
    syy = sum((b - my) ** 2 for b in ry)
    if sxx == 0.0 or syy == 0.0:
        return float("nan")
    return sum((a - mx) * (b - my) for a, b in zip(rx, ry)) / math.sqrt(sxx * syy)


@dataclass
class PrefixStudy:
    """``rho[p]`` = Spearman(``accel_p``, resampled posterior spread) across observations; ``best_prefix`` is its
    argmax (``None`` when no correlation could be formed)."""

    num_resamples: int
    num_observations: int
    divergences: list[float]
    accel_by_prefix: dict[int, list[float]]
    rho: dict[int, float]
    best_prefix: int | None
    default_prefix: int
    rho_at_default: float

    def to_dict(self) -> dict:
        return {"num_resamples": self.num_resamples, "num_observations": self.num_observations,
                "divergences": self.divergences,
                "accel_by_prefix": {str(k): v for k, v in self.accel_by_prefix.items()},
                "rho": {str(k): v for k, v in self.rho.items()}, "best_prefix": self.best_prefix,
                "default_prefix": self.default_prefix, "rho_at_default": self.rho_at_default}


@dataclass
class AccelDiagnosticReport:
    num_steps: int
    prefix: int
    num_scored_dims: list[int]
    max_action_dim: int
    float32_scores: list[float]
    serving_scores: list[float]
    serving_dtype: str
    dtype_floor: float          # median |fp32 - serving| under the same noise
    noise_spread: float         # std over redrawn noise on one observation
    observation_spread: float   # std across observations: the signal
    signal_to_floor: float
    prefix_sweep: dict[int, float] = field(default_factory=dict)
    prefix_study: PrefixStudy | None = None
    observation_source: str = "unspecified"

    def to_dict(self) -> dict:
        d = {k: getattr(self, k) for k in ("num_steps", "prefix", "num_scored_dims", "max_action_dim", "float32_scores",
                                           "serving_scores", "serving_dtype", "dtype_floor", "noise_spread",
                                           "observation_spread", "signal_to_floor", "observation_source")}
        d["prefix_sweep"] = {str(k): v for k, v in self.prefix_sweep.items()}
        d["prefix_study"] = self.prefix_study.to_dict() if self.prefix_study else None
        return d


# ------------------------------------------------------------------------------------------------------ measurements
def fixed_noise(policy, batch_size: int, device, seed: int) -> torch.Tensor:
    """A reproducible draw of the sampler's action shape (production passes ``noise=None``)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    cfg = policy.config
    return torch.randn(batch_size, cfg.chunk_size, cfg.max_action_dim, generator=g, dtype=torch.float32).to(device)


def _cast_batch(policy, batch: dict) -> dict:
    """Floating entries follow the policy's CURRENT parameter dtype (the fp32 leg feeds fp32 frames); masks, indices
    and strings stay as they are."""
    dtype = next(policy.parameters()).dtype
    return {k: (v.to(dtype) if isinstance(v, torch.Tensor) and v.is_floating_point() else v) for k, v in batch.items()}


def score_once(policy, batch: dict, noise: torch.Tensor | None) -> list[float]:
    with torch.inference_mode():
        policy.sample_actions(_cast_batch(policy, batch), noise=noise)
    return list(policy.last_accel or [])


def _dataset_index(policy, obs: dict) -> torch.Tensor:
    state = obs["state"]
    return policy._resolve_dataset_index(obs, state.shape[0], state.device)


def posterior_spread(policy, chunks: list[torch.Tensor], dataset_index: torch.Tensor) -> list[float]:
    """``K`` resampled chunks ``(B, chunk, dim)`` in raw units -> one spread per sample: the root mean square, over
    the scored elements, of the per-element standard deviation across resamples, in normalised units.  The same dim
    mask and executed-row window as the meter, and per-dim standardisation, make it commensurate with ``accel``.  A
    delta-action offset is identical across the resamples of one observation and cancels in the deviation."""
    stacked = torch.stack([c.to(torch.float32) for c in chunks], dim=0)
    width = stacked.shape[-1]
    scale = action_dim_scale(policy.unnormalize_outputs, max_action_dim=width,
                             dataset_index=dataset_index).to(stacked.device)
    dims = resolve_action_dim_mask(policy.unnormalize_outputs, max_action_dim=width,
                                   dataset_index=dataset_index).to(stacked.device)
    deviation = stacked.std(dim=0, unbiased=True) / scale[:, None, :]
    mask = dims.to(torch.float32)[:, None, :].expand_as(deviation).clone()
    mask[:, min(policy.config.n_action_steps, deviation.shape[1]):, :] = 0.0
    total = mask.sum(dim=(1, 2))
    spread = torch.sqrt((deviation.pow(2) * mask).sum(dim=(1, 2)) / total.clamp_min(1.0))
    return [float(s) if n > 0 else float("nan") for s, n in zip(spread.tolist(), total.tolist())]


def resample_observation(policy, batch: dict, dataset_index: torch.Tensor, *, num_resamples: int,
                         seed: int) -> tuple[float, dict[int, float]]:
    """``K`` denoises of one observation with independent noise: (posterior spread, ``{p: mean accel_p}``), both
    averaged over the batch rows.  ``policy.accel_prefix`` must already be the full schedule so that the trace holds
    every prefix."""
    device = next(policy.parameters()).device
    B = batch["state"].shape[0]
    chunks, per_prefix = [], {}
    for k in range(num_resamples):
        noise = fixed_noise(policy, B, device, seed + k)
        with record_traces() as meters, torch.inference_mode():
            chunks.append(policy.sample_actions(_cast_batch(policy, batch), noise=noise).to(torch.float32))
        if not meters:
            raise RuntimeError("accel produced no meter for this resample -- `policy.accel_prefix` must be set before "
                               "calling `resample_observation`.")
        for p, values in meters[-1].prefix_values().items():
            per_prefix.setdefault(p, []).extend(values)
    spreads = posterior_spread(policy, chunks, dataset_index)
    return _mean(spreads), {p: _mean(v) for p, v in per_prefix.items()}


def measure_prefix_quality(policy, observations: list[dict], *, num_resamples: int = 32, seed: int = 0) -> PrefixStudy:
    """Ranks every prefix by how well ``accel_p`` follows the resampled posterior spread.  ``len(observations) * K``
    denoise passes; every prefix comes out of the same passes.  The observations must span a range of real
    uncertainty (frames at a stride through episodes, not repeats of one scene)."""
    if len(observations) < 3:
        raise ValueError(f"the prefix study correlates accel_p against posterior spread across observations, and "
                         f"{len(observations)} of them cannot produce a meaningful rank correlation (any two points "
                         "correlate perfectly). Supply at least 3; 8+ is better.")
    original = policy.accel_prefix
    divergences: list[float] = []
    by_prefix: dict[int, list[float]] = {}
    try:
        policy.accel_prefix = policy.config.num_steps
        for i, obs in enumerate(observations):
            spread, per_prefix = resample_observation(policy, obs, _dataset_index(policy, obs),
                                                      num_resamples=num_resamples, seed=seed + 1000 * i)
            divergences.append(spread)
            for p, v in per_prefix.items():
                by_prefix.setdefault(p, []).append(v)
            logger.info("observation %d/%d: posterior spread %.6g over %d resamples", i + 1, len(observations), spread,
                        num_resamples)
    finally:
        policy.accel_prefix = original
    rho = {p: spearman(v, divergences) for p, v in by_prefix.items()}
    finite = {p: r for p, r in rho.items() if math.isfinite(r)}
    fallback = default_prefix(policy.config.num_steps)
    return PrefixStudy(num_resamples, len(observations), divergences, {p: list(v) for p, v in by_prefix.items()}, rho,
                       max(finite, key=finite.get) if finite else None, fallback, rho.get(fallback, float("nan")))


def signal_to_floor(observation_spread: float, dtype_floor: float) -> float:
    """NaN when the floor was never measured (not the same thing as a floor measured at zero, which gives inf)."""
    if not math.isfinite(dtype_floor):
        return float("nan")
    return observation_spread / dtype_floor if dtype_floor > 0.0 else float("inf")


def diagnose_accel(policy, observations: list[dict], *, num_noise_repeats: int = 8, num_resamples: int = 32,
                   measure_dtype_floor: bool = True, seed: int = 0) -> AccelDiagnosticReport:
    if len(observations) < 2:
        raise ValueError("accel diagnosis needs at least two distinct observations -- the go/no-go compares "
                         "between-observation spread against the rounding floor, and one observation has no spread.")
    if getattr(policy, "_n_candidates", 1) > 1:
        raise ValueError("this diagnostic pins the noise draw and reads one score per observation; best-of-N fans the "
                         "draw out and publishes the selected candidate's score. Run it with n_candidates=1.")
    cfg = policy.config
    device = next(policy.parameters()).device
    serving_dtype = next(policy.parameters()).dtype
    policy.accel_prefix = default_prefix(cfg.num_steps)
    B = observations[0]["state"].shape[0]
    dims = resolve_action_dim_mask(policy.unnormalize_outputs, max_action_dim=cfg.max_action_dim,
                                   dataset_index=_dataset_index(policy, observations[0]))
    num_scored = [int(n) for n in dims.sum(dim=-1).cpu().tolist()]
    logger.info("accel scores %s of %d action dims (the rest have no spread in the norm stats and count as padding)",
                num_scored, cfg.max_action_dim)

    # (1) same field, same noise, two precisions
    noise = fixed_noise(policy, B, device, seed)
    serving = [s for obs in observations for s in score_once(policy, obs, noise)]
    full: list[float] = []
    if measure_dtype_floor:
        logger.info("re-running in float32 to isolate the rounding floor")
        policy.to(dtype=torch.float32)
        try:
            full = [s for obs in observations for s in score_once(policy, obs, noise)]
        finally:
            # not a blanket cast: the SigLIP patch / position tables stay fp32 in a served policy
            to_dtype_preserving_siglip_float32(policy, dtype=serving_dtype)
    else:
        logger.warning("skipping the float32 leg: the dtype floor and the signal/floor ratio will be NaN; run once with "
                       "it enabled to establish the floor of this checkpoint")
    floor = _median([abs(a - b) for a, b in zip(full, serving) if math.isfinite(a) and math.isfinite(b)])

    # (2) one observation, redrawn noise
    repeats = [s for _ in range(num_noise_repeats) for s in score_once(policy, observations[0], None)]

    # (3) every prefix from one pass at the full schedule
    original = policy.accel_prefix
    try:
        policy.accel_prefix = cfg.num_steps
        with record_traces() as meters:
            score_once(policy, observations[0], noise)
        sweep = {p: _mean(v) for p, v in meters[-1].prefix_values().items()}
    finally:
        policy.accel_prefix = original

    # (4) which prefix follows the posterior spread
    study = None
    if num_resamples > 0 and len(observations) >= 3:
        logger.info("prefix quality: %d observations x %d resamples = %d denoise passes", len(observations),
                    num_resamples, len(observations) * num_resamples)
        study = measure_prefix_quality(policy, observations, num_resamples=num_resamples, seed=seed)

    obs_spread = _std(serving)
    return AccelDiagnosticReport(
        num_steps=int(cfg.num_steps), prefix=int(policy.accel_prefix), num_scored_dims=num_scored,
        max_action_dim=int(cfg.max_action_dim), float32_scores=[float(x) for x in full],
        serving_scores=[float(x) for x in serving], serving_dtype=str(serving_dtype).removeprefix("torch."),
        dtype_floor=floor, noise_spread=_std(repeats), observation_spread=obs_spread,
        signal_to_floor=signal_to_floor(obs_spread, floor), prefix_sweep=sweep, prefix_study=study)


# ------------------------------------------------------------------------------------------------------------ report
def prefix_verdict(study: PrefixStudy) -> list[str]:
    if study.best_prefix is None:
        return ["  INCONCLUSIVE -- no prefix produced a computable correlation. Usually every observation shared one "
                "spread value; draw observations from more episodes."]
    best = study.rho[study.best_prefix]
    if best < 0.3:
        return [f"  WEAK -- even the best prefix (p={study.best_prefix}) correlates only rho={best:+.3f} with the "
                "resampled posterior spread on this checkpoint. accel is a poor proxy here whatever the prefix; read "
                "downstream detection numbers as a test of that, not as a tuning problem."]
    lines = [f"  Best prefix p={study.best_prefix} (rho={best:+.3f}); default_prefix would pick "
             f"p={study.default_prefix} (rho={study.rho_at_default:+.3f})."]
    gap = best - study.rho_at_default
    if math.isfinite(gap) and gap > 0.1:
        lines.append(f"  The default gives up {gap:.3f} of rank correlation here. Set "
                     f"`--policy.accel_prefix={study.best_prefix}` for this checkpoint and calibrate any threshold "
                     "under the same prefix (it is part of the provenance).")
    else:
        lines.append("  The default is within noise of the best; no reason to override it on this checkpoint.")
    return lines


def format_report(r: AccelDiagnosticReport) -> str:
    """The thresholds (3x, 10x) are judgement calls: near 1 the score is mostly bf16 rounding, by about 10 rounding
    is a minor perturbation."""
    ratio = r.signal_to_floor
    if math.isnan(ratio):      # first: every comparison against NaN is False and would fall through to "OK"
        verdict = ("NOT MEASURED -- the float32 leg was skipped, so there is no rounding floor to compare the signal "
                   f"against. Re-run once with {DTYPE_FLOOR_ENV}=1 (the floor is fixed per checkpoint).")
    elif ratio < 3.0:
        verdict = ("STOP -- the between-observation spread is within 3x of the pure-rounding floor, so accel here is "
                   "mostly measuring bfloat16 arithmetic. Keep the action projection in float32 before calibrating "
                   "any threshold.")
    elif ratio < 10.0:
        verdict = ("MARGINAL -- real signal exceeds the rounding floor but not comfortably. Expect the certain end of "
                   "the range to be compressed; prefer a float32 action projection if latency allows.")
    else:
        verdict = "OK -- real signal dominates the rounding floor."
    finite_sweep = {p: v for p, v in r.prefix_sweep.items() if math.isfinite(v)}
    top = max(finite_sweep, key=finite_sweep.get) if finite_sweep else None
    bar = "=" * 78
    lines = ["", bar, "accel diagnostic", bar,
             f"  schedule            T = {r.num_steps}, prefix p = {r.prefix}",
             f"  scored action dims  {r.num_scored_dims} of {r.max_action_dim}",
             f"  serving dtype       {r.serving_dtype}",
             f"  observations        {r.observation_source}", "",
             f"  dtype floor         {r.dtype_floor:.6g}   (median |float32 - serving|, same noise)",
             f"  noise spread        {r.noise_spread:.6g}   (std over redrawn noise, one observation)",
             f"  observation spread  {r.observation_spread:.6g}   (std across observations = the signal)",
             f"  signal / floor      {r.signal_to_floor:.2f}", "", f"  {verdict}", "", "  prefix sweep (mean accel_p):"]
    for p, v in sorted(r.prefix_sweep.items()):
        lines.append(f"    p={p:>3}/{r.num_steps}  {v:.6g}{'  <- max' if p == top else ''}")
    lines += ["", "  The largest accel_p is NOT the best prefix: both of its sums accumulate over the prefix, so it rises "
              "with p whether or not the extra steps carry information. The selection criterion is below."]
    s = r.prefix_study
    if s is None:
        lines += ["", f"  No prefix study was run (needs >= 3 observations and resamples > 0), so p = {r.prefix} is the "
                  "default rather than a measurement on this checkpoint."]
    else:
        lines += ["", f"  prefix quality (Spearman rho vs resampled posterior spread, K={s.num_resamples}, "
                  f"n={s.num_observations}):"]
        for p, v in sorted(s.rho.items()):
            marks = (["<- best"] if p == s.best_prefix else []) + (["(default_prefix)"] if p == s.default_prefix else [])
            shown = "   nan" if not math.isfinite(v) else f"{v:+.3f}"
            lines.append(f"    p={p:>3}/{r.num_steps}  rho = {shown}{('  ' + ' '.join(marks)) if marks else ''}")
        lines += [""] + prefix_verdict(s)
    lines.append(bar)
    return "\n".join(lines)


# ------------------------------------------------------------------------------------------------------ observations
def allocate_draws(sizes: list[int], count: int) -> list[int]:
    """Splits ``count`` draws over datasets of the given sizes: each is offered an even share of what is still
    outstanding, capped by what it holds; passes repeat so that a short dataset anywhere in the list is made up by
    the others.  The total is ``min(count, sum(sizes))`` -- asking for fewer draws than datasets never rounds up."""
    quotas = [0] * len(sizes)
    remaining = min(count, sum(sizes))
    while remaining > 0:
        hungry = [i for i, s in enumerate(sizes) if quotas[i] < s]
        if not hungry:
            break
        moved = False
        for pos, i in enumerate(hungry):
            if remaining <= 0:
                break
            take = min(max(1, remaining // (len(hungry) - pos)), remaining, sizes[i] - quotas[i])
            if take > 0:
                quotas[i] += take
                remaining -= take
                moved = True
        if not moved:
            break
    return quotas


def dataset_observations(cfg: TrainPipelineConfig, device, count: int) -> list[dict]:
    """Single-sample observations from the configured mixture, at a stride through every member dataset (adjacent
    frames share a scene and a posterior and would understate the spread).  Preferred over synthetic frames, which
    are out of distribution by construction."""
    from torch.utils.data import DataLoader, Subset

    from ..datasets.factory import make_dataset_mixture
    mixture = make_dataset_mixture(cfg)
    datasets = [d for d in (getattr(mixture, "datasets", None) or [mixture]) if len(d)]
    if not datasets:
        raise ValueError("The configured dataset mixture is empty; cannot draw observations.")
    out: list[dict] = []
    for pos, (ds, want) in enumerate(zip(datasets, allocate_draws([len(d) for d in datasets], count))):
        if want <= 0:
            continue
        stride = max(1, len(ds) // want)
        logger.info("drawing %d observation(s) from dataset %d (%d frames) at stride %d", want, pos, len(ds), stride)
        idx = [min(i * stride, len(ds) - 1) for i in range(want)]
        for batch in DataLoader(Subset(ds, idx), batch_size=1):
            out.append({k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()})
    if len(out) != count:
        logger.warning("requested %d observation(s) but the mixture supplied %d (dataset sizes %s); the rank "
                       "correlations are over the smaller sample", count, len(out), [len(d) for d in datasets])
    return out


def synthetic_observations(cfg: TrainPipelineConfig, device, count: int) -> list[dict]:
    """Noise frames, for when no dataset is reachable: measures the out-of-distribution regime, and the report says so."""
    g = torch.Generator(device="cpu").manual_seed(1234)
    H, W = cfg.resolution
    out = []
    for _ in range(count):
        obs = {"state": torch.randn(1, cfg.max_state_dim, generator=g).to(device), "prompt": ["pick up the object"],
               "img_is_pad": torch.zeros(1, cfg.num_cams, dtype=torch.bool, device=device)}
        for i in range(cfg.num_cams):
            obs[f"camera{i}"] = torch.rand(1, 3, H, W, generator=g).to(device)
        out.append(obs)
    return out


@parser.wrap()
def diagnose_main(cfg: TrainPipelineConfig):
    init_logging()
    from ..policies.candidates import refuse_candidates
    refuse_candidates(cfg, reason="this diagnostic controls the noise draw and reads one score per observation. Run "
                      "it with policy.n_candidates=1.")
    policy = make_policy(cfg.policy)
    policy.eval()
    device = torch.device(getattr(cfg.policy, "device", None) or "cpu")
    policy.to(device)
    to_dtype_preserving_siglip_float32(policy, dtype=torch.bfloat16 if device.type == "cuda" else torch.float32)

    count = int(os.environ.get(OBSERVATIONS_ENV, "24"))
    members = getattr(getattr(cfg, "dataset_mixture", None), "datasets", None)
    if members:
        observations, source = dataset_observations(cfg, device, count), f"{len(members)} configured dataset(s)"
    else:
        logger.warning("no dataset_mixture configured -- falling back to SYNTHETIC noise observations, which are out "
                       "of distribution: the measured spread reflects that regime, not deployment")
        observations, source = synthetic_observations(cfg, device, count), "SYNTHETIC noise (not deployment-representative)"
    report = diagnose_accel(policy, observations, num_resamples=int(os.environ.get(RESAMPLES_ENV, "32")),
                            measure_dtype_floor=os.environ.get(DTYPE_FLOOR_ENV, "1") not in ("0", "false", "False"))
    report.observation_source = source
    print(format_report(report))
    out = Path(cfg.output_dir or ".") / "accel_diagnostic"
    out.mkdir(parents=True, exist_ok=True)
    (out / "report.json").write_text(json.dumps(report.to_dict(), indent=2) + "\n")
    logger.info("wrote %s", out / "report.json")
    return report


def main() -> None:
    diagnose_main()


if __name__ == "__main__":
    main()
