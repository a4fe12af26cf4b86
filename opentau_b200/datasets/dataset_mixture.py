"""Weighted mixture of datasets: tagging, per-dataset normalisation heads, seeded hierarchical sampling.

Behaviour follows the reference (OpenTau ``src/opentau/datasets/dataset_mixture.py:83-1270``): every sample
is tagged with ``dataset_repo_id`` and ``dataset_index`` (the row of the stacked statistics); datasets that
share a normalisation key (repo id + robot type + control mode) share a head; ranks draw from one common
seeded stream and keep their own positions, so sharding needs no communication.
"""

from __future__ import annotations

import logging
from typing import Any, Iterator, Sequence

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset, IterableDataset

from ..configs.types import FeatureType, PolicyFeature
from .sampler import HierarchicalSampler


def compute_norm_key(repo_id: str, robot_type: str | None = None, control_mode: str | None = None) -> str:
    parts = [repo_id]
    if robot_type:
        parts.append(f"robot={robot_type}")
    if control_mode:
        parts.append(f"ctrl={control_mode}")
    return "|".join(parts)


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


def standardized_stats(ds) -> dict:
    """Statistics of one member under the STANDARD feature names (``state``, ``actions``, ``camera{i}``): raw LeRobot
    keys go through the dataset's name map, the column selection is applied, and vectors are zero-padded to the
    pipeline's ``max_state_dim`` / ``max_action_dim`` (a padded dim has zero range, which normalisation maps to 0)."""
    explicit = getattr(ds, "stats", None)
    if explicit:
        return explicit
    raw = getattr(getattr(ds, "meta", None), "stats", None) or {}
    name_map = getattr(ds, "_name_map", None)
    if not raw or not name_map:
        return raw
    out: dict[str, dict[str, np.ndarray]] = {}
    for std, key in name_map.items():
        if key not in raw:
            continue
        st = {k: np.asarray(v, np.float32) for k, v in raw[key].items()}
        index = {"state": getattr(ds, "state_index", None), "actions": getattr(ds, "action_index", None)}.get(std)
        width = {"state": getattr(ds, "max_state_dim", None), "actions": getattr(ds, "max_action_dim", None)}.get(std)
        if std in ("state", "actions"):
            for k, v in list(st.items()):
                if k == "count" or v.ndim != 1:
                    continue
                if index is not None:
                    v = v[np.asarray(index)]
                if width is not None and v.shape[0] < width:
                    v = np.concatenate([v, np.zeros(width - v.shape[0], np.float32)])
                st[k] = v
        out[std] = st
    return out


class DatasetMixtureMetadata:
    """Aggregated view over the members: features, one statistics dict per normalisation head, names."""

    def __init__(self, datasets: Sequence[Dataset], names: Sequence[str], norm_keys: Sequence[str]):
        self.names = list(names)
        self.norm_keys: list[str] = []
        self.dataset_to_norm_index: dict[str, int] = {}
        per_head: dict[str, list[dict]] = {}
        for ds, name, key in zip(datasets, names, norm_keys):
            if key not in per_head:
                per_head[key] = []
                self.norm_keys.append(key)
            per_head[key].append(standardized_stats(ds))
            self.dataset_to_norm_index[name] = self.norm_keys.index(key)
        self.per_dataset_stats = [aggregate_stats(per_head[k]) for k in self.norm_keys]
        self.dataset_names = list(self.norm_keys)
        self.policy_features = self._features(datasets[0])
        self.stats = self.per_dataset_stats[0] if self.per_dataset_stats else {}

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


def aggregate_stats(stats_list: list[dict]) -> dict:
    """Combines the statistics of several datasets that share a head: min of mins, max of maxes, pooled
    mean / std (count-weighted when counts are present), quantiles from the outer envelope."""
    stats_list = [s for s in stats_list if s]
    if not stats_list:
        return {}
    if len(stats_list) == 1:
        return stats_list[0]
    out: dict[str, dict[str, np.ndarray]] = {}
    for key in set().union(*[set(s) for s in stats_list]):
        parts = [s[key] for s in stats_list if key in s]
        counts = np.array([float(np.asarray(p.get("count", 1)).reshape(-1)[0]) for p in parts])
        w = counts / counts.sum()
        agg: dict[str, np.ndarray] = {}
        if all("min" in p for p in parts):
            agg["min"] = np.min([np.asarray(p["min"], np.float32) for p in parts], axis=0)
            agg["max"] = np.max([np.asarray(p["max"], np.float32) for p in parts], axis=0)
        if all("mean" in p for p in parts):
            means = np.stack([np.asarray(p["mean"], np.float32) for p in parts])
            stds = np.stack([np.asarray(p["std"], np.float32) for p in parts])
            wv = w.reshape(-1, *([1] * (means.ndim - 1)))
            mean = (means * wv).sum(0)
            var = ((stds**2 + (means - mean) ** 2) * wv).sum(0)
            agg["mean"], agg["std"] = mean, np.sqrt(var)
        if all("q01" in p for p in parts):
            agg["q01"] = np.min([np.asarray(p["q01"], np.float32) for p in parts], axis=0)
            agg["q99"] = np.max([np.asarray(p["q99"], np.float32) for p in parts], axis=0)
        agg["count"] = np.array([counts.sum()])
        out[key] = agg
    return out


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


class WeightedDatasetMixture:
    def __init__(self, datasets: Sequence[Dataset], names: Sequence[str], weights: Sequence[float] | None = None,
                 norm_keys: Sequence[str] | None = None, seed: int = 1000, action_freq: float | None = None):
        if not datasets:
            raise ValueError("a mixture needs at least one dataset")
        self.weights = list(weights) if weights is not None else [float(len(d)) for d in datasets]
        self.names = list(names)
        norm_keys = list(norm_keys) if norm_keys is not None else list(names)
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
