"""``accel``: a flow-matching uncertainty proxy read off the velocities a sample call already computes.

Over the first ``p`` of ``T`` Euler steps,

    accel_p = p * sum_{t=1}^{p-1} ||v_t - v_{t-1}||  /  sum_{t=0}^{p-1} ||v_t||

A confident flow is a straight line at constant velocity and scores near 0; a flow that bends scores high.  The
cost is two vector norms per denoise step, accumulated in fp32 on the device with no host synchronisation.  Only a
PREFIX of the schedule is scored because the last steps (towards the clean action) are dominated by discretisation
noise; the samplers here integrate noise -> data with the time variable running 1 -> 0, so the prefix is the first
``p`` loop iterations.

Two masks decide whether the number means anything, and both fail silently when they are wrong:

* action dims: the samplers work ``max_action_dim`` wide while an embodiment uses fewer; the padded tail is
  unsupervised network output.  ``real_action_dim`` is a dataset key and does not exist at inference, so
  :func:`resolve_action_dim_mask` recovers the real dims from the action normalisation statistics;
* chunk rows: rows frozen by real-time chunking and rows outside the executed window never reach the robot
  (:func:`executed_row_mask`).

A score is only comparable with scores taken under the same :class:`AccelProvenance`.  The feature is off unless an
entry point arms it through :func:`configure_accel`.  Behavioural reference: ``src/opentau/policies/accel.py:111-863``.
"""

from __future__ import annotations

import contextlib
import contextvars
import logging
import os
from dataclasses import asdict, dataclass, field, fields
from typing import Any, Iterator

import torch
from torch import Tensor

from ..configs.types import NormalizationMode
from .normalize import stat_names_for_mode

logger = logging.getLogger(__name__)

# below this denominator every scored velocity was (near) zero -- the masks removed everything -- and the ratio is
# not a measurement: the meter answers NaN there, because 0.0 would read as "maximally certain"
DENOMINATOR_FLOOR = 1e-12
# a prefix of one velocity has an empty numerator, i.e. 0 for every field: refused, not clamped
MIN_PREFIX = 2
# arms accel on an entry point that has no config field for it: ``auto`` or an integer >= MIN_PREFIX
ACCEL_PREFIX_ENV = "OPENTAU_ACCEL_PREFIX"

# Meters built while a diagnostic runs are handed back through this sink, which doubles as the "keep a per-step
# trace" switch.  A context variable, so that a diagnostic in one thread (or task) never captures the meters of a
# serving thread that calls ``sample_actions`` at the same time.
_TRACE_SINK: contextvars.ContextVar[list | None] = contextvars.ContextVar("accel_trace_sink", default=None)


@contextlib.contextmanager
def record_traces() -> Iterator[list["AccelMeter"]]:
    """Collect the meters built inside this context, each with its per-step trace switched on, so that one denoise
    pass yields the score at every prefix (:meth:`AccelMeter.value_at`).  The previous setting comes back on exit."""
    created: list[AccelMeter] = []
    token = _TRACE_SINK.set(created)
    try:
        yield created
    finally:
        _TRACE_SINK.reset(token)


def _need_schedule(num_steps: int) -> None:
    if num_steps < MIN_PREFIX:
        raise ValueError(f"accel needs at least {MIN_PREFIX} denoise steps to form one velocity difference, "
                         f"but num_steps={num_steps}.")


def default_prefix(num_steps: int) -> int:
    """The online-detector choice ``T - 1`` (never below :data:`MIN_PREFIX`).  A prefix sweep usually peaks nearer
    ``0.4 T - 0.5 T``: this is a sane default, not an optimum, and on the 5-step schedules the two are far apart."""
    _need_schedule(num_steps)
    return max(MIN_PREFIX, num_steps - 1)


def resolve_prefix(prefix: int | None, num_steps: int) -> int | None:
    """``None`` stays off; otherwise the prefix is checked against :data:`MIN_PREFIX` and clamped to the schedule."""
    if prefix is None:
        return None
    if prefix < MIN_PREFIX:
        raise ValueError(f"accel prefix must be >= {MIN_PREFIX} (a shorter prefix has an empty numerator and would "
                         f"report 0.0 for every field), got {prefix}.")
    _need_schedule(num_steps)
    return min(int(prefix), num_steps)


@dataclass(frozen=True)
class AccelProvenance:
    """Everything that shifts the distribution of the score.  A threshold fitted under one provenance says nothing
    about a stream taken under another; keep this beside the values and check with :func:`assert_comparable`.

    ``num_scored_dims`` and ``dataset_index`` vary per sample inside one run and are recorded but not compared.
    ``n_candidates`` is compared: best-of-N publishes the score of the candidate a critic selected, which is not the
    distribution a single draw has."""

    policy_type: str
    num_steps: int
    prefix: int
    chunk_size: int
    n_action_steps: int
    max_delay: int
    action_norm_mode: str
    has_delta_action_map: bool
    velocity_dtype: str
    num_scored_dims: tuple[int, ...] = ()
    dataset_index: tuple[int, ...] = ()
    n_candidates: int = 1

    COMPARABLE_FIELDS = ("policy_type", "num_steps", "prefix", "chunk_size", "n_action_steps", "max_delay",
                         "action_norm_mode", "has_delta_action_map", "velocity_dtype", "n_candidates")

    def to_dict(self) -> dict:
        return asdict(self)

    @classmethod
    def from_dict(cls, payload: dict) -> "AccelProvenance":
        """Inverse of :meth:`to_dict`; keys this version does not know are dropped."""
        known = {f.name for f in fields(cls)}
        kw = {k: v for k, v in payload.items() if k in known}
        for name in ("num_scored_dims", "dataset_index"):
            if kw.get(name) is not None:
                kw[name] = tuple(kw[name])
        return cls(**kw)

    def comparable_with(self, other: "AccelProvenance") -> bool:
        return all(getattr(self, n) == getattr(other, n) for n in self.COMPARABLE_FIELDS)


def assert_comparable(fitted: AccelProvenance, observed: AccelProvenance) -> None:
    """Raises with every disagreeing field named, calibrated value against observed value."""
    diffs = [f"{n}: calibrated on {getattr(fitted, n)!r}, observed {getattr(observed, n)!r}"
             for n in AccelProvenance.COMPARABLE_FIELDS if getattr(fitted, n) != getattr(observed, n)]
    if diffs:
        raise ValueError("accel calibration is not applicable to this stream -- " + "; ".join(diffs)
                         + ". Recalibrate under the deployment configuration.")


# ----------------------------------------------------------------------------------------------- action-dim statistics
def _action_dim_signature(unnormalize: torch.nn.Module, action_key: str) -> tuple[Tensor, NormalizationMode, float]:
    """``(heads, dim)`` spread of the action feature per normalisation head: ``|std|`` under MEAN_STD, ``|hi - lo|``
    under MIN_MAX / QUANTILE (the range, not the divisor).  One reader for the mask and the scale, so that both see
    the same buffer, stat names and live ``eps``."""
    feature = getattr(unnormalize, "features", {}).get(action_key)
    if feature is None:
        raise ValueError(f"accel: no feature {action_key!r} on the policy's Unnormalize; cannot derive the "
                         "action-dim mask.")
    mode = getattr(unnormalize, "norm_map", {}).get(feature.type, NormalizationMode.IDENTITY)
    if isinstance(mode, str):
        mode = NormalizationMode(mode)
    if mode is NormalizationMode.IDENTITY:
        raise ValueError("accel: ACTION normalization is IDENTITY, so no stats buffer exists and the "
                         "padded-action-dim mask cannot be derived. IDENTITY also leaves per-dim scale heterogeneous, "
                         "which violates the estimator's standardized-dimension premise. Disable accel for this "
                         "checkpoint or serve with MEAN_STD.")
    buf = getattr(unnormalize, "buffer_" + action_key.replace(".", "_"), None)
    if buf is None:
        raise ValueError(f"accel: Unnormalize has no stats buffer for {action_key!r}.")
    if mode is NormalizationMode.MEAN_STD:
        sig = buf["std"].detach().abs()
    else:
        lo, hi = stat_names_for_mode(mode)
        sig = (buf[hi].detach() - buf[lo].detach()).abs()
    return sig.reshape(sig.shape[0], -1), mode, float(unnormalize.eps)


def _fit_width(per_head: Tensor, width: int, pad_value) -> Tensor:
    have = per_head.shape[1]
    if have < width:
        pad = torch.full((per_head.shape[0], width - have), pad_value, dtype=per_head.dtype, device=per_head.device)
        return torch.cat([per_head, pad], dim=1)
    return per_head[:, :width]


def _head_rows(dataset_index: Tensor, per_head: Tensor) -> Tensor:
    return dataset_index.to(device=per_head.device, dtype=torch.long).reshape(-1).clamp(0, per_head.shape[0] - 1)


def action_dim_scale(unnormalize: torch.nn.Module, *, max_action_dim: int, dataset_index: Tensor,
                     action_key: str = "actions") -> Tensor:
    """``(B, max_action_dim)`` fp32 divisor that takes raw actions into the normalised space the score lives in
    (``std`` under MEAN_STD, half the range otherwise).  Degenerate and padded dims come back as 1 so that a caller
    can divide unconditionally; the dim mask excludes them anyway."""
    sig, mode, eps = _action_dim_signature(unnormalize, action_key)
    scale = sig.to(torch.float32)
    if mode is not NormalizationMode.MEAN_STD:
        scale = scale / 2.0
    scale = torch.where(torch.isfinite(scale) & (scale >= eps), scale, torch.ones_like(scale))
    per_head = _fit_width(scale, max_action_dim, 1.0)
    return per_head.index_select(0, _head_rows(dataset_index, per_head))


def resolve_action_dim_mask(unnormalize: torch.nn.Module, *, max_action_dim: int, dataset_index: Tensor,
                            action_key: str = "actions") -> Tensor:
    """``(B, max_action_dim)`` bool: dims whose statistics show a spread.  A padded column is constant across the
    dataset, so its ``std`` / range is zero.  This is a heuristic that errs towards dropping signal: a real but
    constant dim (a locked joint) is masked as well, which is harmless for a curvature ratio.  Resolved per
    normalisation head, so two samples of a mixture can score different numbers of dims."""
    sig, mode, eps = _action_dim_signature(unnormalize, action_key)
    head_mask = _fit_width(torch.isfinite(sig) & (sig >= eps), max_action_dim, False)
    rows = _head_rows(dataset_index, head_mask)
    per_sample = head_mask.index_select(0, rows)
    if not bool(per_sample.any()):
        # usually a routing problem, not a broken checkpoint: a mixture carries a placeholder head with all-zero
        # statistics and an observation without provenance falls back to head 0
        per_head = [int(n) for n in head_mask.sum(dim=1).tolist()]
        usable = [i for i, n in enumerate(per_head) if n > 0]
        hint = (f" Head(s) {usable} do have usable stats -- tag the observation with its dataset (repo id, or robot "
                "type and control mode) so that it is routed there instead of falling back to head 0."
                if usable else " No head has usable action stats; this checkpoint cannot support accel.")
        raise ValueError(f"accel: every action dim of norm head(s) {sorted({int(i) for i in rows.tolist()})} is "
                         f"degenerate in the {mode.name} stats, so the score would be computed over zero dimensions. "
                         f"Scorable dims per head: {per_head}." + hint)
    return per_sample


# --------------------------------------------------------------------------------------------------------------- meter
@dataclass
class AccelMeter:
    """Running accumulator for one sample call.  It is passed through the sampler as an argument rather than kept
    on the module, so no state survives a call or crosses threads::

        meter.set_row_mask(rows)        # (B | 1, chunk) bool, before the loop
        for each Euler step:
            v_t = denoise_step(...)
            meter.update(v_t)           # before the step is taken
    """

    prefix: int
    batch_size: int
    device: torch.device
    dim_mask: Tensor | None = None
    record_trace: bool = False
    _num: Tensor = field(init=False, repr=False)
    _den: Tensor = field(init=False, repr=False)
    _prev: Tensor | None = field(default=None, init=False, repr=False)
    _mask: Tensor | None = field(default=None, init=False, repr=False)
    _steps: int = field(default=0, init=False)
    _trace: list = field(default_factory=list, init=False, repr=False)

    def __post_init__(self) -> None:
        if self.prefix < MIN_PREFIX:
            raise ValueError(f"accel prefix must be >= {MIN_PREFIX}, got {self.prefix}.")
        self._num = torch.zeros(self.batch_size, dtype=torch.float32, device=self.device)
        self._den = torch.zeros(self.batch_size, dtype=torch.float32, device=self.device)
        if self.dim_mask is not None:
            self._mask = self.dim_mask.to(torch.float32)[:, None, :]

    def set_row_mask(self, row_mask: Tensor) -> None:
        """Score only these chunk rows; multiplies with the dim mask.  Call once, before the loop."""
        rows = row_mask.to(torch.float32)[:, :, None]
        self._mask = rows if self._mask is None else rows * self._mask

    def update(self, v_t: Tensor) -> None:
        """Adds one step's velocity ``(B, chunk, dim)``; a no-op once ``prefix`` steps are in."""
        if self._steps >= self.prefix:
            return
        v = v_t.to(torch.float32)
        if self._mask is not None:
            v = v * self._mask
        v = v.flatten(1)
        self._den = self._den + torch.linalg.vector_norm(v, dim=1)
        if self._prev is not None:
            self._num = self._num + torch.linalg.vector_norm(v - self._prev, dim=1)
        self._prev = v
        self._steps += 1
        if self.record_trace:
            self._trace.append((self._num, self._den))

    @property
    def steps(self) -> int:
        """Velocities accumulated so far (short of ``prefix`` when the schedule was)."""
        return self._steps

    @staticmethod
    def _ratio(count: int, num: Tensor, den: Tensor) -> Tensor:
        nan = torch.full_like(den, float("nan"))
        return torch.where(den > DENOMINATOR_FLOOR, count * num / den.clamp_min(DENOMINATOR_FLOOR), nan)

    def value(self) -> Tensor:
        """``(B,)`` fp32 score with the number of accumulated velocities as the multiplier.  NaN where it is
        undefined: fewer than two velocities, or everything masked out."""
        if self._steps < MIN_PREFIX:
            return torch.full_like(self._den, float("nan"))
        return self._ratio(self._steps, self._num, self._den)

    def value_at(self, prefix: int) -> Tensor:
        """The score this call would have reported at a shorter prefix (needs the trace: build the meter inside
        :func:`record_traces`).  Both sums are running sums, so one pass serves every prefix."""
        if not self.record_trace:
            raise RuntimeError("AccelMeter.value_at requires record_trace=True -- build the meter inside "
                               "`record_traces()`.")
        if not MIN_PREFIX <= prefix <= self._steps:
            raise ValueError(f"prefix must be in [{MIN_PREFIX}, {self._steps}] for this meter, got {prefix}.")
        num, den = self._trace[prefix - 1]
        return self._ratio(prefix, num, den)

    def prefix_values(self) -> dict[int, list[float]]:
        return {p: [float(x) for x in self.value_at(p).detach().to("cpu", torch.float32).tolist()]
                for p in range(MIN_PREFIX, self._steps + 1)}

    def to_list(self) -> list[float]:
        """Plain floats: a tensor made under ``inference_mode`` stays an inference tensor even after a clone, and a
        detector that later updates it in place would raise."""
        return [float(x) for x in self.value().detach().to("cpu", torch.float32).tolist()]


def make_meter(policy: torch.nn.Module, *, batch_size: int, device, dataset_index: Tensor | None = None,
               max_action_dim: int | None = None) -> AccelMeter | None:
    """The meter for one sample call, or ``None`` while ``policy.accel_prefix`` is unset.  The dim mask comes from
    ``policy.unnormalize_outputs``; an IDENTITY-normalised action feature is refused."""
    prefix = getattr(policy, "accel_prefix", None)
    if prefix is None:
        return None
    cfg = policy.config
    prefix = resolve_prefix(int(prefix), cfg.num_steps)
    device = torch.device(device)
    if dataset_index is None:
        dataset_index = torch.zeros(batch_size, dtype=torch.long, device=device)
    dim_mask = resolve_action_dim_mask(policy.unnormalize_outputs,
                                       max_action_dim=max_action_dim or cfg.max_action_dim,
                                       dataset_index=dataset_index).to(device)
    sink = _TRACE_SINK.get()
    meter = AccelMeter(prefix, batch_size, device, dim_mask, record_trace=sink is not None)
    if sink is not None:
        sink.append(meter)
    return meter


def build_provenance(policy: torch.nn.Module, meter: AccelMeter, *, dataset_index: Tensor | None = None,
                     velocity_dtype: torch.dtype | None = None, n_candidates: int = 1) -> AccelProvenance:
    cfg = policy.config
    mode = (cfg.normalization_mapping or {}).get("ACTION")
    if velocity_dtype is None:
        velocity_dtype = next(policy.parameters()).dtype
    scored = () if meter.dim_mask is None else tuple(int(n) for n in meter.dim_mask.sum(dim=-1).cpu().tolist())
    index = () if dataset_index is None else tuple(int(i) for i in dataset_index.detach().cpu().reshape(-1).tolist())
    return AccelProvenance(
        policy_type=getattr(cfg, "type", type(cfg).__name__), num_steps=int(cfg.num_steps), prefix=int(meter.prefix),
        chunk_size=int(cfg.chunk_size), n_action_steps=int(cfg.n_action_steps),
        max_delay=int(getattr(cfg, "max_delay", 0) or 0), action_norm_mode=getattr(mode, "name", str(mode)),
        has_delta_action_map=bool(getattr(cfg, "delta_action_state_map", None)),
        velocity_dtype=str(velocity_dtype).removeprefix("torch."), num_scored_dims=scored, dataset_index=index,
        n_candidates=int(n_candidates))


def configure_accel(policy: torch.nn.Module, cfg: Any = None, *, override: int | str | None = None) -> int | None:
    """The one switch every serving entry point uses.  First non-``None`` wins: ``override`` (the entry point's own
    flag), ``cfg.policy.accel_prefix``, ``$OPENTAU_ACCEL_PREFIX``.  Nothing requested leaves the policy untouched and
    the sampler's accel lines dead.  Call it before the warm-up calls, so that a checkpoint that cannot support the
    score (IDENTITY actions, no usable dims) fails at start-up rather than on the first request.

    Returns the resolved prefix or ``None``; raises when accel is requested but the policy has no ``accel_prefix``
    attribute (its sampler is not wired for it), no ``num_steps`` schedule, or the prefix is invalid."""
    requested: int | str | None = override
    pol_cfg = getattr(cfg, "policy", None) if cfg is not None else None
    if requested is None and pol_cfg is not None:
        requested = getattr(pol_cfg, "accel_prefix", None)
    if requested is None:
        requested = os.environ.get(ACCEL_PREFIX_ENV)
    if requested is None or (isinstance(requested, str) and not requested.strip()):
        return None
    policy_type = getattr(pol_cfg, "type", None) or getattr(policy.config, "type", type(policy).__name__)
    if not hasattr(policy, "accel_prefix"):
        raise ValueError(f"accel was requested ({requested!r}) but policy type {policy_type!r} does not expose "
                         "`accel_prefix`, i.e. its sampler is not wired for denoising acceleration.")
    num_steps = getattr(policy.config, "num_steps", None)
    if num_steps is None:
        raise ValueError(f"accel was requested ({requested!r}) but policy type {policy_type!r} has no `num_steps` "
                         "denoise schedule to read velocities off.")
    text = str(requested).strip().lower()
    if text == "auto":
        prefix = default_prefix(num_steps)
    else:
        try:
            prefix = resolve_prefix(int(text), num_steps)
        except ValueError as exc:
            if "invalid literal" in str(exc):
                raise ValueError(f"accel prefix must be an integer >= {MIN_PREFIX} or the literal 'auto', "
                                 f"got {requested!r}.") from exc
            raise
    policy.accel_prefix = prefix
    logger.info("accel enabled: prefix=%d of num_steps=%d (requested %r)", prefix, num_steps, requested)
    return prefix


def executed_row_mask(*, prefix_mask: Tensor, delay: Tensor | int, chunk_size: int, n_action_steps: int,
                      device) -> Tensor:
    """Rows a sampler should score: not frozen by real-time chunking, and inside the window that is executed,
    ``[delay, delay + n_action_steps)`` -- not ``[0, n_action_steps)``, which is wrong whenever ``delay > 0``."""
    positions = torch.arange(chunk_size, device=device)[None, :]
    if isinstance(delay, Tensor):
        horizon = (delay.reshape(-1, 1) if delay.ndim else delay).to(device) + n_action_steps
    else:
        horizon = int(delay) + n_action_steps
    return (~prefix_mask.to(device)) & (positions < horizon)


def publish(policy, meter: AccelMeter | None, *, dataset_index: Tensor | None, n_candidates: int = 1,
            selected: Tensor | None = None) -> None:
    """Writes ``last_accel`` (one value per observation), ``last_accel_provenance`` and, under best-of-N,
    ``last_accel_candidates`` (the full grid) on the policy.  With candidates the published value is the selected
    candidate's: consumers such as the gRPC reply read ``last_accel[0]`` and expect one entry per observation."""
    if meter is None:
        return
    values = meter.to_list()
    if n_candidates <= 1:
        policy.last_accel = values
        policy.last_accel_candidates = None
        policy.last_accel_provenance = build_provenance(policy, meter, dataset_index=dataset_index)
        return
    chosen = [int(i) for i in selected.detach().cpu().reshape(-1).tolist()]
    policy.last_accel_candidates = [values[b * n_candidates:(b + 1) * n_candidates] for b in range(len(chosen))]
    policy.last_accel = [values[b * n_candidates + c] for b, c in enumerate(chosen)]
    policy.last_accel_provenance = build_provenance(policy, meter, dataset_index=dataset_index,
                                                    n_candidates=n_candidates)
