"""Dataset construction from the pipeline config (reference ``src/opentau/datasets/factory.py:258-784``).

``make_dataset`` builds one member (LeRobot on disk, a VQA corpus, or the synthetic generator) and, when a
validation ratio is set, its deterministic episode-level train/val split; ``make_dataset_mixture`` assembles the
weighted mixture(s) with one normalisation head per usable ``(robot_type, control_mode)`` pair.
"""

from __future__ import annotations

import logging
from pathlib import Path
from typing import Any

import numpy as np
import torch

from ..configs.default import DatasetConfig
from .dataset_mixture import WeightedDatasetMixture
from .lerobot_dataset import LeRobotDataset, LeRobotDatasetMetadata
from .standard_data_format_mapping import get_mapping
from .transforms import ImageTransforms


def resolve_delta_timestamps(cfg, dataset_cfg: DatasetConfig, ds_meta: LeRobotDatasetMetadata) -> dict[str, list[float]]:
    """Per raw feature, the time offsets to fetch: the action chunk at ``action_freq`` (policy's
    ``action_delta_indices``), and ``n_obs_history`` past frames for cameras and state."""
    action_freq = cfg.dataset_mixture.action_freq or ds_meta.fps
    name_map = get_mapping(dataset_cfg.repo_id, ds_meta.features, dataset_cfg.data_features_name_mapping)
    reverse = {v: k for k, v in name_map.items()}
    out: dict[str, list[float]] = {}
    for key in ds_meta.features:
        std = reverse.get(key)
        if std is None:
            continue
        if std == "actions":
            idx = cfg.policy.action_delta_indices if cfg.policy is not None else list(range(cfg.action_chunk))
            if idx is not None:
                out[key] = [i / action_freq for i in idx]
        elif "camera" in std or std == "state":
            n_obs = cfg.dataset_mixture.n_obs_history
            if n_obs is not None:
                interval = getattr(cfg.policy, "history_interval", 1)
                out[key] = [-(n_obs - 1 - i) * interval / action_freq for i in range(n_obs)]
            else:
                out[key] = [0.0]
    return out


def val_split_generator(seed: int | None, repo_id: str) -> np.random.Generator:
    """The split depends only on (seed, dataset name), so it is identical on every rank and after a resume."""
    import zlib
    return np.random.default_rng([0 if seed is None else int(seed), zlib.crc32(repo_id.encode())])


def split_episodes(episodes: list[int], ratio: float, seed: int | None, repo_id: str) -> tuple[list[int], list[int]]:
    if not ratio or len(episodes) < 2:
        return list(episodes), []
    perm = val_split_generator(seed, repo_id).permutation(len(episodes))
    n_val = min(len(episodes) - 1, max(1, int(round(len(episodes) * ratio))))
    val = sorted(episodes[i] for i in perm[:n_val])
    train = sorted(episodes[i] for i in perm[n_val:])
    return train, val


def warn_if_resumed_split_differs(output_dir: Path, splits: dict[str, list[int]]) -> None:
    """Stores the validation episodes next to the checkpoints; on resume a different split is reported loudly."""
    import json
    f = Path(output_dir) / "val_split.json"
    if f.exists():
        old = json.loads(f.read_text())
        if old != splits:
            logging.warning("validation split differs from the one this run started with (%s)", f)
    else:
        f.parent.mkdir(parents=True, exist_ok=True)
        f.write_text(json.dumps(splits))


class SyntheticDataset(torch.utils.data.Dataset):
    """Random samples of fixed shapes (benchmarks and smoke runs): ``synthetic: {length, state_dim, action_dim}``."""

    def __init__(self, cfg, spec: dict[str, Any]):
        self.cfg, self.spec = cfg, spec
        self.length = int(spec.get("length", 1024))
        self.repo_id = f"synthetic:{spec.get('name', 'default')}"
        sd, ad = int(spec.get("state_dim", 8)), int(spec.get("action_dim", 8))
        self.sd, self.ad = sd, ad
        one = lambda n, d: np.concatenate([np.ones(d, np.float32), np.zeros(n - d, np.float32)])  # noqa: E731
        self.stats = {
            "state": {"min": -3 * one(cfg.max_state_dim, sd), "max": 3 * one(cfg.max_state_dim, sd),
                      "mean": np.zeros(cfg.max_state_dim, np.float32), "std": one(cfg.max_state_dim, sd),
                      "count": np.array([self.length])},
            "actions": {"min": -3 * one(cfg.max_action_dim, ad), "max": 3 * one(cfg.max_action_dim, ad),
                        "mean": np.zeros(cfg.max_action_dim, np.float32), "std": one(cfg.max_action_dim, ad),
                        "count": np.array([self.length])}}

    def __len__(self) -> int:
        return self.length

    def __getitem__(self, i: int) -> dict:
        cfg = self.cfg
        g = torch.Generator().manual_seed(int(i))
        H, W = cfg.resolution
        out: dict[str, Any] = {}
        T = cfg.dataset_mixture.n_obs_history
        for c in range(cfg.num_cams):
            shape = (T, 3, H, W) if T else (3, H, W)
            out[f"camera{c}"] = (torch.randint(0, 256, shape, generator=g, dtype=torch.uint8).float() / 255).to(torch.bfloat16)
        st = torch.zeros((T, cfg.max_state_dim) if T else (cfg.max_state_dim,))
        st[..., :self.sd] = torch.randn(*st.shape[:-1], self.sd, generator=g)
        ac = torch.zeros(cfg.action_chunk, cfg.max_action_dim)
        ac[:, :self.ad] = torch.randn(cfg.action_chunk, self.ad, generator=g)
        out.update(state=st.to(torch.bfloat16), actions=ac.to(torch.bfloat16), prompt=f"synthetic task {i % 7}",
                   response="", img_is_pad=torch.zeros(cfg.num_cams, dtype=torch.bool),
                   action_is_pad=torch.zeros(cfg.action_chunk, dtype=torch.bool),
                   obs_history_is_pad=torch.zeros(T or 1, dtype=torch.bool),
                   real_action_dim=torch.tensor(self.ad), advantage=torch.tensor(0.0, dtype=torch.bfloat16),
                   return_bin_idx=torch.tensor(i % 7), return_continuous=torch.tensor(-(i % 7) / 7.0),
                   source=self.repo_id, episode_index=int(i) // 100, frame_index=int(i) % 100)
        return out


def make_dataset(dataset_cfg: DatasetConfig, cfg, return_advantage_input: bool = False):
    """Returns the dataset, or ``(train, val)`` when a validation ratio applies."""
    ratio = dataset_cfg.val_split_ratio if dataset_cfg.val_split_ratio is not None else cfg.dataset_mixture.val_split_ratio
    want_val = bool(ratio) and cfg.val_freq > 0
    if dataset_cfg.synthetic is not None:
        ds = SyntheticDataset(cfg, dataset_cfg.synthetic)
        if want_val:
            spec_val = {**dataset_cfg.synthetic, "length": max(1, int(ds.length * ratio))}
            return ds, SyntheticDataset(cfg, spec_val)
        return ds
    if dataset_cfg.vqa is not None:
        from .vqa import make_vqa_dataset
        ds = make_vqa_dataset(dataset_cfg.vqa, cfg)
        if want_val:
            return ds, make_vqa_dataset(dataset_cfg.vqa, cfg, train=False)
        return ds
    meta = LeRobotDatasetMetadata(dataset_cfg.repo_id, root=dataset_cfg.root, revision=dataset_cfg.revision)
    delta = resolve_delta_timestamps(cfg, dataset_cfg, meta)
    tfs = ImageTransforms(dataset_cfg.image_transforms) if dataset_cfg.image_transforms.enable else None
    episodes = sorted(dataset_cfg.episodes if dataset_cfg.episodes is not None else meta.episodes)
    if dataset_cfg.excluded_episodes:
        episodes = [e for e in episodes if e not in set(dataset_cfg.excluded_episodes)]
    mix = cfg.dataset_mixture
    kw = dict(root=dataset_cfg.root, delta_timestamps=delta,
              tolerance_s=dataset_cfg.tolerance_s if dataset_cfg.tolerance_s is not None else mix.tolerance_s,
              revision=dataset_cfg.revision, video_backend=dataset_cfg.video_backend,
              image_resample_strategy=mix.image_resample_strategy, vector_resample_strategy=mix.vector_resample_strategy,
              dataset_cfg=dataset_cfg, meta=meta, return_advantage_input=return_advantage_input)
    if mix.require_non_empty_robot_type and not (dataset_cfg.robot_type or meta.robot_type):
        raise ValueError(f"dataset {dataset_cfg.repo_id} has no robot_type")
    if mix.require_non_empty_control_mode and not (dataset_cfg.control_mode or meta.control_mode):
        raise ValueError(f"dataset {dataset_cfg.repo_id} has no control_mode")
    if want_val:
        tr, va = split_episodes(episodes, ratio, cfg.seed, dataset_cfg.repo_id)
        train = LeRobotDataset(cfg, dataset_cfg.repo_id, episodes=tr, image_transforms=tfs, **kw)
        if not va:
            return train
        val = LeRobotDataset(cfg, dataset_cfg.repo_id, episodes=va, image_transforms=None,
                             train=mix.val_enable_optional_key_dropout, **kw)
        # the two switches of the validation subset are independent of each other
        val.enable_prompt_substitution = mix.val_enable_prompt_substitution
        attach_delta_action_stats(train, dataset_cfg, cfg)
        val.delta_action_stats = train.delta_action_stats      # validation is normalised like training
        return train, val
    ds = LeRobotDataset(cfg, dataset_cfg.repo_id, episodes=episodes, image_transforms=tfs, **kw)
    attach_delta_action_stats(ds, dataset_cfg, cfg)
    return ds


def attach_delta_action_stats(dataset: LeRobotDataset, dataset_cfg: DatasetConfig, cfg) -> None:
    """A delta-action dataset's stored statistics describe ABSOLUTE per-frame actions; the training targets are
    displacements from the chunk-start state, typically several times narrower.  Their statistics are computed from
    the numeric columns the dataset already holds in memory (cached under the dataset's root, keyed by everything that
    changes them) and replace ``state`` / ``actions`` in the mixture's pooled statistics
    (reference ``src/opentau/datasets/factory.py:112-235``)."""
    dataset.delta_action_stats = None
    if not dataset.delta_action_state_map:
        return
    from .delta_action_stats import compute_delta_stats_from_columns, delta_stats_cache_key, load_or_compute_delta_stats
    name_map = dataset._get_name_map()
    a_key, s_key = name_map["actions"], name_map["state"]
    # the action horizon in frames (mean offsets: with a jittered horizon the statistics describe its centre)
    offsets = np.asarray(dataset.delta_timestamps.get(a_key, [0.0]), np.float64) * dataset.fps
    max_rows = cfg.dataset_mixture.delta_stats_max_rows
    logging.info("%s: delta joint actions on; stored map %s -> post-index map %s (state_index=%s, action_index=%s)",
                 dataset_cfg.repo_id, dataset_cfg.delta_action_state_map, dataset.delta_action_state_map,
                 dataset_cfg.state_index, dataset_cfg.action_index)
    key = delta_stats_cache_key(state_index=dataset_cfg.state_index, action_index=dataset_cfg.action_index,
                                delta_map=dataset.delta_action_state_map, chunk_offsets=offsets,
                                vector_resample_strategy=dataset.vector_resample_strategy, episodes=dataset.episodes,
                                excluded_episodes=dataset_cfg.excluded_episodes, fps=dataset.fps,
                                revision=dataset_cfg.revision, max_rows=max_rows)

    def compute():
        num = dataset._numeric
        return compute_delta_stats_from_columns(
            num[s_key].numpy(), num[a_key].numpy(), num["episode_index"].numpy(),
            delta_map=dataset.delta_action_state_map, chunk_offsets=offsets, state_index=dataset_cfg.state_index,
            action_index=dataset_cfg.action_index, strategy=dataset.vector_resample_strategy, max_rows=max_rows)

    dataset.delta_action_stats = load_or_compute_delta_stats(dataset.root, key, compute)


def dedup_names(names: list[str]) -> list[str]:
    """Mixture-level names: the second and later entries of one repository get ``#1``, ``#2``, ... appended, so the
    name -> head table and the per-dataset validation buckets keep one row per entry."""
    seen: dict[str, int] = {}
    out = []
    for n in names:
        k = seen.get(n, 0)
        seen[n] = k + 1
        out.append(n if k == 0 else f"{n}#{k}")
    return out


def make_dataset_mixture(cfg, return_advantage_input: bool = False):
    """``WeightedDatasetMixture`` or ``(train_mixture, val_mixture)``."""
    mix = cfg.dataset_mixture
    if not mix.datasets:
        raise ValueError("dataset_mixture.datasets is empty")
    trains, vals, names, val_names, val_w = [], [], [], [], []
    weights = list(mix.weights) if mix.weights else None
    for i, dcfg in enumerate(mix.datasets):
        res = make_dataset(dcfg, cfg, return_advantage_input)
        tr, va = res if isinstance(res, tuple) else (res, None)
        if dcfg.stats is not None:
            tr.stats = {k: {s: np.asarray(v, np.float32) for s, v in d.items()} for k, d in dcfg.stats.items()}
        trains.append(tr), names.append(dcfg.name)
        if va is not None:
            vals.append(va), val_names.append(dcfg.name)
            val_w.append(weights[i] if weights else float(len(va)))
    seed = cfg.seed if cfg.seed is not None else 0
    names, val_names = dedup_names(names), dedup_names(val_names)
    # heads come from each member's (robot_type, control_mode), config overrides included; the validation split takes
    # the TRAINING split's rows, so a validation batch is normalised exactly like a training batch of that dataset
    train_mix = WeightedDatasetMixture(trains, names, weights, seed=seed, action_freq=mix.action_freq)
    if vals:
        by_name = dict(zip(names, [train_mix.meta.norm_keys[train_mix.meta.dataset_to_norm_index[n]] for n in names]))
        return train_mix, WeightedDatasetMixture(vals, val_names, val_w, [by_name.get(n, n) for n in val_names],
                                                 seed=seed + 1, action_freq=mix.action_freq)
    return train_mix
