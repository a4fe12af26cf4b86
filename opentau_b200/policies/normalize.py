"""Per-sample input/target normalisation with one row of statistics per dataset ("norm head").

Statistics live in frozen parameters ``buffer_<feature>.<stat>`` shaped ``(num_heads, *feat)``
so they ride along in ``model.safetensors`` under the reference's key names
(OpenTau ``src/opentau/policies/normalize.py:296-717``).  Semantics kept:

* MEAN_STD: ``(x - mean) / (std + eps)`` with ``|std| < eps`` snapped to 1;
* MIN_MAX / QUANTILE: ``[lo, hi] -> [-1, 1]``; a zero-range dim maps to 0 when
  ``zero_range_center`` (new checkpoints) and to -1 otherwise (legacy);
* buffers start at ``+inf`` and the first use asserts they were filled.
"""

from __future__ import annotations

import logging

import numpy as np
import torch
from torch import Tensor, nn

from ..configs.types import FeatureType, NormalizationMode, PolicyFeature

OPENPI_EPS = 1e-6
LEGACY_EPS = 1e-8
EPS = OPENPI_EPS

_STATS_OF_MODE = {
    NormalizationMode.MEAN_STD: ("mean", "std"),
    NormalizationMode.MIN_MAX: ("min", "max"),
    NormalizationMode.QUANTILE: ("q01", "q99"),
}


def stat_names_for_mode(mode: NormalizationMode) -> tuple[str, str]:
    return _STATS_OF_MODE[mode]


def _mode_of(norm_map: dict, ft: PolicyFeature) -> NormalizationMode:
    m = norm_map.get(ft.type, None)
    if m is None:
        m = norm_map.get(ft.type.value, NormalizationMode.IDENTITY)
    return NormalizationMode(m)


def resolve_stat_row(ds_stats: dict, key: str, name: str):
    """``stats[key][name]``; a missing statistic is an error.  QUANTILE deliberately does NOT fall back to min / max: one
    dataset's row would then sit on another scale than its peers, the very thing quantile normalisation exists to avoid.
    A row can also lack quantiles because it is a pooled head whose members disagree (the aggregation drops a quantile
    that not every member carries and names the members that lack it)."""
    if key not in ds_stats:
        raise KeyError(f"no stats for feature '{key}' (available: {list(ds_stats)})")
    entry = ds_stats[key]
    if name in entry:
        return entry[name]
    hint = ""
    if name.startswith("q") and name[1:].isdigit():
        hint = ("; QUANTILE normalisation needs quantile statistics: recompute this dataset's statistics with quantiles "
                "(for a pooled head, those of the datasets named in the earlier 'dropped from the aggregate' warning), "
                "or map the feature to MIN_MAX / MEAN_STD")
    raise KeyError(f"stats for '{key}' lack '{name}' (available: {list(entry)}){hint}")


#: raw-unit |value - centre| above which a snapped (zero-variance) dim counts as a real deviation worth a warning;
#: <= 0 switches the warning (and its host synchronisation) off.  The snap itself always runs.
SNAP_WARN_TOL = 1e-2
_WARNED_SNAPS: dict[tuple[str, int], float] = {}      # (feature, dim) -> largest deviation already warned about


def warn_snapped_deviation(key: str, snapped: Tensor, deviation: Tensor, dataset_index: Tensor | None,
                           dataset_names: list[str] | None) -> None:
    """A std (or range) of ~0 marks a constant / padding dim and is replaced by 1, so that a value which DEVIATES from
    the constant cannot be divided by ~eps into ~1e6.  On a truly constant dim the deviation is 0 and nothing changes;
    a real deviation means stale statistics or a value zeroed upstream, and is reported once per (feature, dim), again
    only for a larger deviation, with the dataset of the worst sample
    (reference ``src/opentau/policies/normalize.py:76-144``)."""
    trigger = snapped & (deviation.abs() > SNAP_WARN_TOL)
    if not bool(trigger.any()):
        return
    mag = (deviation.abs() * trigger).reshape(-1, deviation.shape[-1]) if deviation.dim() > 1 else (deviation.abs() * trigger)[None]
    per_dim = mag.amax(0)
    fresh = []
    for d in torch.nonzero(per_dim > 0).flatten().tolist():
        v = float(per_dim[d])
        if v > _WARNED_SNAPS.get((key, d), -1.0):
            _WARNED_SNAPS[(key, d)] = v
            fresh.append(d)
    if not fresh:
        return
    worst = max(fresh, key=lambda d: float(per_dim[d]))
    who = None
    if dataset_names is not None and dataset_index is not None and deviation.dim() > 1:
        col = (deviation.abs() * trigger)[..., worst].reshape(deviation.shape[0], -1).amax(1)
        row = int(dataset_index.reshape(-1)[int(col.argmax())])
        who = dataset_names[row] if 0 <= row < len(dataset_names) else None
    logging.warning("zero-variance guard: feature '%s' dim(s) %s have std / range ~ 0, yet a value deviates from the "
                    "constant by up to %.3g (raw units, dataset=%s).  The divisor was set to 1, so nothing blows up, but "
                    "this almost always means stale statistics or a value zeroed upstream: inspect this feature's stats.",
                    key, fresh, float(per_dim[worst]), who)


def warn_missing_keys(features: dict, batch: dict, mode: str) -> None:
    """One line per expected feature that the batch lacks (the feature is then passed over, not an error)."""
    for k in sorted(set(features) - set(batch)):
        if (mode, k) not in _WARNED_MISSING:
            _WARNED_MISSING.add((mode, k))
            logging.warning("'%s' was missing from the batch during %s", k, mode)


_WARNED_MISSING: set[tuple[str, str]] = set()


def _as_f32(v) -> Tensor:
    if isinstance(v, Tensor):
        return v.detach().to(torch.float32).cpu()
    return torch.from_numpy(np.asarray(v, dtype=np.float32))


def create_stats_buffers(features: dict[str, PolicyFeature], norm_map: dict,
                         per_dataset_stats: list[dict] | None = None, num_datasets: int | None = None,
                         dataset_names: list[str] | None = None) -> dict[str, nn.ParameterDict]:
    if per_dataset_stats is None and num_datasets is None:
        raise ValueError("create_stats_buffers needs per_dataset_stats or num_datasets")
    if per_dataset_stats is not None:
        if len(per_dataset_stats) == 0:
            raise ValueError("per_dataset_stats must contain at least one dataset")
        if num_datasets is not None and num_datasets != len(per_dataset_stats):
            raise ValueError(f"num_datasets ({num_datasets}) disagrees with len(per_dataset_stats) "
                             f"({len(per_dataset_stats)})")
        n = len(per_dataset_stats)
    else:
        n = int(num_datasets)
        if n <= 0:
            raise ValueError(f"num_datasets must be positive, got {n}")
    out: dict[str, nn.ParameterDict] = {}
    for key, ft in features.items():
        mode = _mode_of(norm_map, ft)
        if mode is NormalizationMode.IDENTITY:
            continue
        shape = tuple(ft.shape)
        if ft.type is FeatureType.VISUAL:
            if len(shape) != 3 or not (shape[0] < shape[1] and shape[0] < shape[2]):
                raise ValueError(f"{key}: expected a channel-first image shape, got {shape}")
            shape = (shape[0], 1, 1)
        params = {}
        for name in stat_names_for_mode(mode):
            if per_dataset_stats is None:
                t = torch.full((n, *shape), torch.inf, dtype=torch.float32)
            else:
                rows = []
                for i, st in enumerate(per_dataset_stats):
                    label = dataset_names[i] if dataset_names else f"dataset[{i}]"
                    try:
                        row = _as_f32(resolve_stat_row(st, key, name))
                    except KeyError as e:
                        raise KeyError(f"{label}: {e.args[0]}") from None
                    if tuple(row.shape) != shape:
                        raise ValueError(f"{label}['{key}']['{name}'] has shape {tuple(row.shape)}, expected {shape}")
                    rows.append(row)
                t = torch.stack(rows, 0)
            params[name] = nn.Parameter(t, requires_grad=False)
        out[key] = nn.ParameterDict(params)
    return out


def _rows(stat: Tensor, index: Tensor, like: Tensor) -> Tensor:
    g = stat.index_select(0, index.to(stat.device))
    extra = like.ndim - g.ndim
    if extra < 0:
        raise ValueError(f"stats rank {g.ndim} exceeds batch rank {like.ndim}")
    if extra:
        g = g.reshape(g.shape[0], *((1,) * extra), *g.shape[1:])
    return g


class _StatsModule(nn.Module):
    inverse = False

    def __init__(self, features: dict[str, PolicyFeature], norm_map: dict,
                 per_dataset_stats: list[dict] | None = None, dataset_names: list[str] | None = None,
                 num_datasets: int | None = None, zero_range_center: bool = False, eps: float = EPS):
        super().__init__()
        self.features, self.norm_map = features, norm_map
        self.zero_range_center, self.eps = zero_range_center, eps
        self.dataset_names = list(dataset_names) if dataset_names is not None else None
        if per_dataset_stats is not None and dataset_names is not None and len(per_dataset_stats) != len(dataset_names):
            raise ValueError("per_dataset_stats and dataset_names must have the same length")
        for key, buf in create_stats_buffers(features, norm_map, per_dataset_stats, num_datasets,
                                             dataset_names).items():
            setattr(self, "buffer_" + key.replace(".", "_"), buf)

    def _apply(self, fn, recurse=True):
        # statistics stay fp32 whatever the model is cast to
        def keep(t):
            o = fn(t)
            return o.to(torch.float32) if o.is_floating_point() and o.dtype != torch.float32 else o
        return super()._apply(keep, recurse)

    def _watch_snap(self, key: str, snapped: Tensor, deviation: Tensor, idx: Tensor) -> None:
        """Reports a deviation on a snapped dim WITHOUT stalling the launch queue: on a GPU the one-bit verdict is
        copied to pinned memory behind an event and read at a later call, once the event has passed; only a positive
        verdict (the rare, broken case) pays for the detailed message.  On the CPU the check is immediate."""
        if deviation.device.type != "cuda":
            warn_snapped_deviation(key, snapped, deviation, idx, self.dataset_names)
            return
        if torch.cuda.is_current_stream_capturing():      # a captured graph must hold no host-side bookkeeping
            return
        pending = self.__dict__.setdefault("_snap_pending", [])
        for item in list(pending):
            if item[0].query():
                pending.remove(item)
                if bool(item[1].item()):
                    warn_snapped_deviation(item[2], item[3], item[4], item[5], self.dataset_names)
        if len(pending) >= 8:               # the device is far behind: do not pile up references
            return
        flag = torch.empty(1, dtype=torch.bool, pin_memory=True)
        flag.copy_((snapped & (deviation.abs() > SNAP_WARN_TOL)).any().reshape(1), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        pending.append((ev, flag, key, snapped, deviation, idx))

    def _snapping_possible(self) -> bool:
        """Whether any buffer has a zero-variance dim at all (cached at the first forward pass): the healthy common
        case then pays neither the check nor its host synchronisation.  A zero-variance dim that arrives later (a
        statistics injection after the first pass) is still snapped, only not reported."""
        cached = getattr(self, "_snap_active", None)
        if cached is not None:
            return cached
        active = False
        for key, ft in self.features.items():
            mode = _mode_of(self.norm_map, ft)
            buf = getattr(self, "buffer_" + key.replace(".", "_"), None)
            if buf is None or mode is NormalizationMode.IDENTITY:
                continue
            a_name, b_name = stat_names_for_mode(mode)
            spread = buf[b_name] if mode is NormalizationMode.MEAN_STD else buf[b_name] - buf[a_name]
            if bool((torch.isfinite(spread) & (spread.abs() < self.eps)).any()):
                active = True
                break
        self._snap_active = active
        return active

    @property
    def num_heads(self) -> int:
        for p in self.parameters():
            return p.shape[0]
        return 1

    @torch.no_grad()
    def forward(self, batch: dict[str, Tensor], dataset_index: Tensor | None = None) -> dict[str, Tensor]:
        warn_missing_keys(self.features, batch, "unnormalization" if self.inverse else "normalization")
        batch = dict(batch)
        for key, ft in self.features.items():
            if key not in batch:
                continue
            mode = _mode_of(self.norm_map, ft)
            if mode is NormalizationMode.IDENTITY:
                continue
            x = batch[key]
            if x.numel() == 0:
                continue
            buf = getattr(self, "buffer_" + key.replace(".", "_"))
            idx = dataset_index
            if idx is None:
                idx = torch.zeros(x.shape[0], dtype=torch.long, device=x.device)
            a_name, b_name = stat_names_for_mode(mode)
            a, b = _rows(buf[a_name], idx, x), _rows(buf[b_name], idx, x)
            if torch.isinf(a).any() or torch.isinf(b).any():
                raise AssertionError(
                    f"`{a_name}`/`{b_name}` of '{key}' is infinity: initialise with per_dataset_stats, "
                    "call policy._inject_stats(...), or load a checkpoint that has the normalization buffers")
            xf = x.to(torch.float32)
            watch = (not self.inverse and SNAP_WARN_TOL > 0 and not torch.compiler.is_compiling()
                     and not torch.onnx.is_in_onnx_export() and self._snapping_possible())
            if mode is NormalizationMode.MEAN_STD:
                std = torch.where(b.abs() < self.eps, torch.ones_like(b), b)
                y = xf * (std + self.eps) + a if self.inverse else (xf - a) / (std + self.eps)
                if watch:
                    self._watch_snap(key, (b.abs() < self.eps).expand_as(xf), xf - a, idx)
            else:
                rng = b - a
                den = torch.where(rng.abs() < self.eps, torch.ones_like(rng), rng)
                if watch:
                    self._watch_snap(key, (rng.abs() < self.eps).expand_as(xf), xf - a, idx)
                if self.inverse:
                    y = (xf + 1) / 2 * (den + self.eps) + a
                    if self.zero_range_center:
                        y = y - 0.5 * (den - rng)
                else:
                    shifted = xf - a
                    if self.zero_range_center:
                        shifted = shifted + 0.5 * (den - rng)
                    y = shifted / (den + self.eps) * 2 - 1
            batch[key] = y.to(x.dtype) if x.is_floating_point() else y
        return batch


class Normalize(_StatsModule):
    inverse = False


class Unnormalize(_StatsModule):
    inverse = True
