"""Weighted mixture of datasets: tagging, per-dataset normalisation heads, seeded hierarchical sampling.

Behaviour follows the reference (OpenTau ``src/opentau/datasets/dataset_mixture.py:83-1270``): every sample
is tagged with ``dataset_repo_id`` and ``dataset_index`` (the row of the stacked statistics); datasets that
share a usable ``(robot_type, control_mode)`` pair share a head (others get one of their own); ranks draw from one common
seeded stream and keep their own positions, so sharding needs no communication.
"""

from __future__ import annotations

import logging
from typing import Any, Iterator, Sequence

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset, IterableDataset

from ..configs.types import FeatureType, PolicyFeature
from .compute_stats import QUANTILE_STAT_NAMES, aggregate_stats as _aggregate_stats
from .sampler import HierarchicalSampler


#: tag values that mean "not recorded": they must not anchor an ``unknown::<mode>`` head shared by unrelated robots
_MISSING_TAG_VALUES = frozenset({"unknown"})
_PER_DIM_STATS = ("mean", "std", "min", "max") + QUANTILE_STAT_NAMES


def compute_norm_key(robot_type: str | None, control_mode: str | None, fallback_name: str) -> tuple[str, bool]:
    """``("<robot_type>::<control_mode>", False)`` (original casing), or ``(fallback_name, True)`` when either tag is
    ``None``, blank, or ``"unknown"`` in any casing.

    Datasets of one robot under one control mode share units, axis count and physical ranges, so they share one
    normalisation head; a dataset without usable tags still gets a head, keyed by its own name and shared with
    nobody (reference ``src/opentau/datasets/dataset_mixture.py:171-207``)."""
    rt, cm = (robot_type or "").strip(), (control_mode or "").strip()
    if not rt or not cm or rt.casefold() in _MISSING_TAG_VALUES or cm.casefold() in _MISSING_TAG_VALUES:
        return fallback_name, True
    return f"{rt}::{cm}", False


class _TaggedDataset(Dataset):
    """Adds the mixture tags to every sample of a member dataset."""

    def __init__(self, dataset: Dataset, repo_id: str, norm_index: int):
        self.dataset, self.repo_id, self.norm_index = dataset, repo_id, norm_index

    def __len__(self) -> int:
        return len(self.dataset)

    def __getitem__(self, i: int) -> dict[str, Any]:
        item = dict(self.dataset[i])
        item["dataset_repo_id"] = self.repo_id
        item["dataset_index"] = torch.tensor(self.norm_index, dtype=torch.long)
        return item


def _placeholder_camera_stats(count) -> dict[str, np.ndarray]:
    st = {"min": np.zeros((3, 1, 1), np.float32), "max": np.ones((3, 1, 1), np.float32),
          "mean": np.zeros((3, 1, 1), np.float32), "std": np.zeros((3, 1, 1), np.float32)}
    if count is not None:                    # v2.0 statistics carry no count; mirror it only where there is one
        st["count"] = np.array(count)
    return st


def standardized_stats(ds) -> dict:
    """Statistics of one member under the STANDARD feature names (``state``, ``actions``, ``camera{i}``), laid out
    like the vectors ``__getitem__`` emits (reference ``dataset_mixture.py:602-775``).

    * raw LeRobot keys go through the dataset's own name map (prompt / response / advantage / mistake / success have
      no statistics; cameras beyond ``num_cams`` are dropped); a mapped key without statistics is an error;
    * a delta-action dataset's precomputed statistics (post-index space) replace ``state`` / ``actions`` wholesale:
      the stored ones describe absolute per-frame actions, the wrong distribution once the transform is on;
    * otherwise ``state_index`` / ``action_index`` select the columns of every per-dim statistic, BEFORE padding,
      in the data path's order;
    * vectors are zero-padded to ``max_state_dim`` / ``max_action_dim`` (a padded dim has zero range: normalisation
      maps it to 0); cameras the dataset lacks get the identity record min 0 / max 1 / mean 0 / std 0;
    * ``mean / std / min / max`` must all be present; non-finite entries of vector features are reported with the
      dataset and the dims (the aggregator leaves those dims of this contributor out)."""
    explicit = getattr(ds, "stats", None)
    if explicit:
        return explicit
    raw = getattr(getattr(ds, "meta", None), "stats", None) or {}
    name_map = getattr(ds, "_name_map", None)
    if not raw or not name_map:
        return raw
    who = getattr(ds, "repo_id", None) or type(ds).__name__
    num_cams = getattr(ds, "num_cams", None)
    out: dict[str, dict[str, np.ndarray]] = {}
    for std, key in name_map.items():
        if std in ("prompt", "response", "advantage", "mistake", "success"):
            continue
        if std.startswith("camera") and num_cams is not None and int(std[len("camera"):]) >= num_cams:
            continue
        if key not in raw:
            if std in ("state", "actions"):
                raise KeyError(f"{who}: no statistics for '{key}' (mapped to '{std}'); available: {sorted(raw)}")
            continue
        out[std] = {k: np.asarray(v, np.float32 if k != "count" else None) for k, v in raw[key].items()}
    delta_stats = getattr(ds, "delta_action_stats", None) or {}
    for std, index, width in (("state", getattr(ds, "state_index", None), getattr(ds, "max_state_dim", None)),
                              ("actions", getattr(ds, "action_index", None), getattr(ds, "max_action_dim", None))):
        if std in delta_stats:
            out[std] = {k: np.asarray(v) for k, v in delta_stats[std].items()}
            index = None                                      # computed from the already-selected columns
        if std not in out:
            continue
        for k, v in list(out[std].items()):
            if k not in _PER_DIM_STATS or v.ndim != 1:
                continue
            if index is not None:
                bad = [i for i in index if i >= v.shape[0]]
                if bad:
                    raise IndexError(f"{who}: {std}_index names column(s) {bad}, but the '{k}' statistic has "
                                     f"{v.shape[0]} column(s)")
                v = v[np.asarray(index)]
            if width is not None and v.shape[0] < width:
                v = np.concatenate([v, np.zeros(width - v.shape[0], v.dtype)])
            out[std][k] = v
    count = out.get("state", {}).get("count")
    for c in range(num_cams or 0):
        out.setdefault(f"camera{c}", _placeholder_camera_stats(count))
    for std, st in out.items():
        missing = {"mean", "std", "min", "max"} - set(st)
        if missing:
            raise KeyError(f"the dataset {who} lacks required statistics of '{std}': {sorted(missing)}")
        if std.startswith("camera"):
            continue
        for k in ("mean", "std", "min", "max", "q01", "q99"):
            if k in st:
                bad = np.flatnonzero(~np.isfinite(np.asarray(st[k], np.float64).ravel()))
                if bad.size:
                    logging.warning("dataset %r: non-finite values in %s.%s at flat indices %s; these dims are left out "
                                    "of the pooled statistics", who, std, k, bad[:16].tolist())
    return out


def _raw_dims(ds, stats: dict) -> tuple[int | None, int | None]:
    """(state width, action width) BEFORE padding: from the dataset's sample contract when it states one, else from
    the column selection, else from the stored statistics."""
    out = []
    for feat, index_attr, raw_key in (("state", "state_index", "state"), ("actions", "action_index", "actions")):
        index = getattr(ds, index_attr, None)
        if index is not None:
            out.append(len(index))
            continue
        meta_stats = getattr(getattr(ds, "meta", None), "stats", None) or {}
        key = (getattr(ds, "_name_map", None) or {}).get(raw_key)
        arr = (meta_stats.get(key) or {}).get("mean") if key else None
        out.append(int(np.asarray(arr).shape[-1]) if arr is not None and np.asarray(arr).ndim else None)
    return out[0], out[1]


class DatasetMixtureMetadata:
    """Aggregated view over the members (reference ``dataset_mixture.py:226-600``).

    ``norm_keys[r]`` names row ``r`` of the policy's stacked statistics; ``per_norm_key_stats[r]`` fills it.  A head
    is shared by every dataset with the same usable ``(robot_type, control_mode)``; the members' statistics are
    pooled with their FRAME totals as weights (sample-count pooling: the mixture's sampling weights would confuse
    "what the data looks like" with "how often it is drawn").  Members that share a real pair must agree on the raw
    (pre-padding) state and action widths.  ``dataset_to_norm_index`` maps a dataset NAME to its row, so inference can
    resolve a ``dataset_repo_id`` even when several datasets share a head; ``norm_key_to_dataset_names`` is the
    reverse listing.  ``delta_action_state_map`` is the one post-index map all delta-action members agree on
    (``None``: absolute actions); the policy stores it to turn its outputs back into absolute actions.

    ``norm_keys`` may be handed in (one per dataset, e.g. by a tool that regroups heads by hand); otherwise they come
    from each member's ``robot_type`` / ``control_mode`` attributes, which already include the config overrides."""

    def __init__(self, datasets: Sequence[Dataset], names: Sequence[str], norm_keys: Sequence[str] | None = None):
        if len(datasets) != len(names):
            raise ValueError(f"{len(datasets)} datasets but {len(names)} names")
        self.names = list(names)
        stats = [standardized_stats(ds) for ds in datasets]
        fallbacks: list[str] = []
        if norm_keys is None:
            per_ds_keys = []
            for ds, name in zip(datasets, names):
                key, fell_back = compute_norm_key(getattr(ds, "robot_type", None), getattr(ds, "control_mode", None), name)
                per_ds_keys.append(key)
                if fell_back:
                    fallbacks.append(name)
        else:
            per_ds_keys = list(norm_keys)
            if len(per_ds_keys) != len(names):
                raise ValueError(f"{len(per_ds_keys)} norm keys but {len(names)} datasets")
        self.norm_keys: list[str] = list(dict.fromkeys(per_ds_keys))
        self.norm_key_to_index: dict[str, int] = {k: i for i, k in enumerate(self.norm_keys)}
        self.dataset_to_norm_index: dict[str, int] = {n: self.norm_key_to_index[k] for n, k in zip(names, per_ds_keys)}
        self.norm_key_to_dataset_names: dict[str, list[str]] = {k: [] for k in self.norm_keys}
        for n, k in zip(names, per_ds_keys):
            self.norm_key_to_dataset_names[k].append(n)
        dims = [_raw_dims(ds, st) for ds, st in zip(datasets, stats)]
        self.per_norm_key_stats: list[dict] = []
        for k in self.norm_keys:
            members = [i for i, dk in enumerate(per_ds_keys) if dk == k and stats[i]]
            if len({dims[i] for i in members}) > 1:
                who = [f"{names[i]} (state_dim={dims[i][0]}, action_dim={dims[i][1]})" for i in members]
                raise ValueError(f"datasets that share the norm key {k!r} have different raw (pre-padding) state / "
                                 f"action widths, so their statistics cannot be pooled: {who}.  Override "
                                 "`DatasetConfig.robot_type` or `control_mode` to give them separate heads.")
            if not members:
                self.per_norm_key_stats.append({})
            elif len(members) == 1:
                self.per_norm_key_stats.append(stats[members[0]])
            else:
                frames = [float(self._total_frames(datasets[i])) for i in members]
                self.per_norm_key_stats.append(_aggregate_stats(
                    [stats[i] for i in members], weights=frames, contributor_names=[names[i] for i in members],
                    context=f"norm head {k!r}"))
        if fallbacks:
            logging.warning("%d dataset(s) have no usable (robot_type, control_mode) pair and get a normalisation head "
                            "of their own, keyed by name; set DatasetConfig.robot_type / control_mode (or fix info.json) "
                            "to share statistics across datasets: %s%s", len(fallbacks), fallbacks[:10],
                            f", ... and {len(fallbacks) - 10} more" if len(fallbacks) > 10 else "")
        lines = [f"normalisation heads: {len(self.norm_keys)} over {len(names)} dataset(s)"]
        for k in sorted(self.norm_keys):
            ds_list = self.norm_key_to_dataset_names[k]
            lines.append(f"  - {k}: {ds_list[:10]}" + (f", ... and {len(ds_list) - 10} more" if len(ds_list) > 10 else ""))
        logging.info("\n".join(lines))
        self.delta_action_state_map = self._resolve_delta_map(datasets, names)
        # the policy factory reads these two names
        self.per_dataset_stats = self.per_norm_key_stats
        self.dataset_names = list(self.norm_keys)
        self.policy_features = self._features(datasets[0])
        self.stats = self.per_norm_key_stats[0] if self.per_norm_key_stats else {}

    def aggregated_action_stats(self, weights: Sequence[float] | None = None) -> dict[str, np.ndarray]:
        """ONE set of action statistics for the whole mixture (the few consumers that need a single range, such as a
        tokenizer fitted under global normalisation).  Heads without ``actions`` are left out together with their
        weight, so the parallel lists cannot slip against each other."""
        w = list(weights) if weights is not None else [1.0] * len(self.per_norm_key_stats)
        rows = [({"actions": s["actions"]}, wi, k) for s, wi, k in zip(self.per_norm_key_stats, w, self.norm_keys)
                if s and "actions" in s]
        if not rows:
            raise ValueError("no head of the mixture has 'actions' statistics")
        if len(rows) == 1:
            return dict(rows[0][0]["actions"])
        return _aggregate_stats([r[0] for r in rows], weights=[r[1] for r in rows],
                                contributor_names=[r[2] for r in rows], context="mixture-wide action statistics")["actions"]

    @staticmethod
    def _total_frames(ds) -> int:
        info = getattr(getattr(ds, "meta", None), "info", None) or {}
        return int(info.get("total_frames") or 0) or max(len(ds), 1)

    @staticmethod
    def _resolve_delta_map(datasets: Sequence[Dataset], names: Sequence[str]) -> dict[int, int] | None:
        """The policy applies ONE inverse transform to every chunk it emits and has no per-sample signal for the
        convention that produced it: robot datasets must be all-delta (with one and the same resolved map, whatever
        their stored layouts) or all-absolute.  Question-answer datasets emit no action chunk and are exempt."""
        maps = [dict(getattr(ds, "delta_action_state_map", None) or {}) for ds in datasets]
        on = [(n, m) for n, m in zip(names, maps) if m]
        if not on:
            return None
        absolute = [n for n, m, ds in zip(names, maps, datasets) if not m and not getattr(ds, "is_vqa", False)]
        if absolute:
            raise ValueError(f"{len(on)} dataset(s) of this mixture use delta joint actions but {len(absolute)} robot "
                             f"dataset(s) do not ({absolute[:10]}); set use_delta_joint_actions consistently "
                             "(question-answer datasets are exempt)")
        first_name, first = on[0]
        differ = [f"{n} -> {m}" for n, m in on[1:] if m != first]
        if differ:
            raise ValueError("datasets disagree on the resolved (post-index) delta_action_state_map, so the policy's "
                             f"inverse would be ambiguous: {first_name} -> {first}, but {differ[:10]}; use state_index / "
                             "action_index to bring them onto one layout")
        logging.info("delta joint actions on for all %d robot dataset(s); post-index map %s", len(on), first)
        return {int(a): int(b) for a, b in first.items()}

    @staticmethod
    def _features(ds: Dataset) -> dict[str, PolicyFeature]:
        feats = getattr(ds, "policy_features", None)
        if feats:
            return dict(feats)
        sample = ds[0]
        out: dict[str, PolicyFeature] = {}
        for k, v in sample.items():
            if not isinstance(v, torch.Tensor):
                continue
            if k.startswith("camera"):
                out[k] = PolicyFeature(FeatureType.VISUAL, tuple(v.shape[-3:]))
            elif k == "state":
                out[k] = PolicyFeature(FeatureType.STATE, (v.shape[-1],))
            elif k == "actions":
                out[k] = PolicyFeature(FeatureType.ACTION, (v.shape[-1],))
        return out


def aggregate_stats(stats_list: list[dict], weights: list[float] | None = None, **kw) -> dict:
    """Statistics of several datasets that share a head (see ``compute_stats.aggregate_stats``); empty records are
    skipped and a single record is returned as it is."""
    keep = [i for i, s in enumerate(stats_list) if s]
    if not keep:
        return {}
    if len(keep) == 1:
        return stats_list[keep[0]]
    return _aggregate_stats([stats_list[i] for i in keep], None if weights is None else [weights[i] for i in keep], **kw)


def collate_standard(samples: list[dict[str, Any]]) -> dict[str, Any]:
    """Stacks tensors, keeps strings as lists; keys missing from some samples are dropped."""
    keys = set(samples[0])
    for s in samples[1:]:
        keys &= set(s)
    out: dict[str, Any] = {}
    for k in sorted(keys):
        v0 = samples[0][k]
        if isinstance(v0, torch.Tensor):
            out[k] = torch.stack([s[k] for s in samples])
        elif isinstance(v0, (int, float, bool, np.integer, np.floating)):
            out[k] = torch.tensor([s[k] for s in samples])
        else:
            out[k] = [s[k] for s in samples]
    return out


class _MixtureStream(IterableDataset):
    def __init__(self, concat: "WeightedDatasetMixture", rank: int, world: int):
        self.m, self.rank, self.world = concat, rank, world

    def __iter__(self) -> Iterator[dict[str, Any]]:
        info = torch.utils.data.get_worker_info()
        wid, nw = (info.id, info.num_workers) if info is not None else (0, 1)
        sampler = HierarchicalSampler(self.m.lengths, self.m.weights, self.m.seed, rank=self.rank * nw + wid,
                                      world=self.world * nw)
        for gi in sampler:
            yield self.m.get_global(gi)


class _SequentialShard(Dataset):
    """Every ``world``-th sample of the concatenated mixture, starting at ``rank``: each sample is visited once."""

    def __init__(self, mixture: "WeightedDatasetMixture", rank: int, world: int):
        self.m, self.rank, self.world = mixture, rank, world

    def __len__(self) -> int:
        n = len(self.m)
        return (n - self.rank + self.world - 1) // self.world if n > self.rank else 0

    def __getitem__(self, i: int) -> dict[str, Any]:
        return self.m.get_global(self.rank + i * self.world)


class WeightedDatasetMixture:
    def __init__(self, datasets: Sequence[Dataset], names: Sequence[str], weights: Sequence[float] | None = None,
                 norm_keys: Sequence[str] | None = None, seed: int = 1000, action_freq: float | None = None):
        if not datasets:
            raise ValueError("a mixture needs at least one dataset")
        self.weights = list(weights) if weights is not None else [float(len(d)) for d in datasets]
        self.names = list(names)
        self.meta = DatasetMixtureMetadata(datasets, names, norm_keys)
        self.datasets = [_TaggedDataset(d, n, self.meta.dataset_to_norm_index[n]) for d, n in zip(datasets, names)]
        self.lengths = [len(d) for d in self.datasets]
        self.offsets = np.concatenate([[0], np.cumsum(self.lengths)[:-1]])
        self.seed, self.action_freq = seed, action_freq

    def __len__(self) -> int:
        return int(sum(self.lengths))

    @property
    def num_frames(self) -> int:
        return len(self)

    def get_global(self, gi: int) -> dict[str, Any]:
        d = int(np.searchsorted(self.offsets, gi, side="right") - 1)
        return self.datasets[d][gi - int(self.offsets[d])]

    def get_dataloader(self, batch_size: int, num_workers: int = 0, rank: int = 0, world: int = 1,
                       prefetch_factor: int | None = None, pin_memory: bool | None = None) -> DataLoader:
        pin = torch.cuda.is_available() if pin_memory is None else pin_memory
        kw: dict[str, Any] = {}
        if num_workers > 0:
            kw.update(prefetch_factor=prefetch_factor or 2, persistent_workers=True)
        return DataLoader(_MixtureStream(self, rank, world), batch_size=batch_size, num_workers=num_workers,
                          collate_fn=collate_standard, pin_memory=pin, drop_last=True, **kw)

    def get_combined_val_dataloader(self, batch_size: int, num_workers: int = 0, rank: int = 0, world: int = 1,
                                    prefetch_factor: int | None = None) -> DataLoader | None:
        """ONE deterministic sequential loader over the whole mixture (validation): no shuffling, no dropped tail,
        every sample scored exactly once, and every rank's shard is full even when a member has fewer frames than
        there are ranks (one loader per dataset would leave most ranks idle on small members, member after member).
        Each sample carries ``dataset_index`` / ``dataset_repo_id``, so the caller can split the metrics per head and
        per dataset afterwards.  ``None`` for an empty mixture
        (reference ``src/opentau/datasets/dataset_mixture.py:1229-1270``)."""
        if len(self) == 0:
            logging.info("combined validation loader skipped: the mixture is empty")
            return None
        kw: dict[str, Any] = {}
        if num_workers > 0:
            kw.update(prefetch_factor=prefetch_factor or 2)
        return DataLoader(_SequentialShard(self, rank, world), batch_size=batch_size, shuffle=False,
                          num_workers=num_workers, collate_fn=collate_standard, pin_memory=torch.cuda.is_available(),
                          drop_last=False, **kw)

    def get_per_dataset_dataloaders(self, batch_size: int, num_workers: int = 0,
                                    prefetch_factor: int | None = None) -> dict[str, DataLoader]:
        """One sequential loader per member (per-dataset evaluation: each member once, in order); empty members are
        skipped (reference ``dataset_mixture.py:1194-1227``)."""
        kw: dict[str, Any] = {}
        if num_workers > 0:
            kw.update(prefetch_factor=prefetch_factor or 2)
        out: dict[str, DataLoader] = {}
        for name, ds in zip(self.names, self.datasets):
            if len(ds) == 0:
                logging.info("no per-dataset loader for the empty dataset %r", name)
                continue
            out[name] = DataLoader(ds, batch_size=batch_size, shuffle=False, num_workers=num_workers,
                                   collate_fn=collate_standard, pin_memory=torch.cuda.is_available(), drop_last=False, **kw)
        return out
