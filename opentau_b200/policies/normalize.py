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
    """Fetches ``stats[key][name]``; QUANTILE falls back to min/max when quantiles are absent."""
    if key not in ds_stats:
        raise KeyError(f"no stats for feature '{key}'")
    entry = ds_stats[key]
    if name in entry:
        return entry[name]
    fallback = {"q01": "min", "q99": "max"}.get(name)
    if fallback and fallback in entry:
        return entry[fallback]
    raise KeyError(f"stats for '{key}' lack '{name}'")


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

    @property
    def num_heads(self) -> int:
        for p in self.parameters():
            return p.shape[0]
        return 1

    @torch.no_grad()
    def forward(self, batch: dict[str, Tensor], dataset_index: Tensor | None = None) -> dict[str, Tensor]:
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
            if mode is NormalizationMode.MEAN_STD:
                std = torch.where(b.abs() < self.eps, torch.ones_like(b), b)
                y = xf * (std + self.eps) + a if self.inverse else (xf - a) / (std + self.eps)
            else:
                rng = b - a
                den = torch.where(rng.abs() < self.eps, torch.ones_like(rng), rng)
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
