"""LeRobot-format datasets: metadata, random-access reader (codebase v2.0 / v2.1 / v3.0) and v2.1 recorder.

Behaviour follows the reference (``src/opentau/datasets/lerobot_dataset.py:184-3321``):

* rows are addressed by a global frame index over the selected episodes; per-feature *delta timestamps* turn
  into soft (fractional) row offsets at the dataset's fps, clipped to the episode with ``<key>_is_pad`` flags, and
  are resampled ``nearest`` or ``linear`` (vectors only);
* camera frames come from parquet-embedded images or from mp4 files (decoded on OpenCV here);
* ``_to_standard_data_format`` renames features to ``camera{i} / state / actions / prompt / response``, resizes
  images with padding to the pipeline resolution, applies column indices and delta actions, zero-pads vectors to
  ``max_state_dim / max_action_dim``, emits the pad masks, optional keys with their dropout rolls, bf16 floats and
  provenance.

The table backend is pyarrow (all parquet files of the selected episodes are concatenated into one in-memory
table; numeric columns are materialised as torch tensors once), not HF ``datasets``.
"""

from __future__ import annotations

import contextlib
import functools
import io
import logging
import random
import shutil
from pathlib import Path
from typing import Any, Callable

import numpy as np
import torch
from torch import Tensor

from .. import ops
from .action_indexing import apply_column_index, resolve_delta_map, subtract_chunk_start_state
from .compute_stats import aggregate_stats, compute_episode_stats, sample_indices
from .hub_transfer import HubTransferMixin
from .standard_data_format_mapping import get_mapping
from .utils import (CODEBASE_VERSION, DEFAULT_CHUNK_SIZE, DEFAULT_FEATURES, DEFAULT_IMAGE_PATH, DEFAULT_PARQUET_PATH,
                    DEFAULT_VIDEO_PATH, EPISODES_PATH, EPISODES_STATS_PATH, INFO_PATH, TASKS_PATH, append_jsonlines,
                    check_timestamps_sync, check_version_compatibility, get_episode_data_index, get_version, load_episodes,
                    load_episodes_stats, load_info, load_stats, load_tasks, serialize_stats, validate_episode_buffer,
                    validate_frame, write_json)
from .video_utils import decode_video_frames, encode_video_frames

HF_HOME = Path.home() / ".cache" / "huggingface" / "lerobot"


def retry_random_on_failure(fn: Callable) -> Callable:
    """``__getitem__`` decorator: on a decode / IO failure, retry a few random indices before giving up."""

    @functools.wraps(fn)
    def wrapped(self, idx):
        n = int(getattr(self, "_getitem_retries", 3))
        last: Exception | None = None
        for attempt in range(n + 1):
            try:
                return fn(self, idx)
            except (OSError, ValueError, RuntimeError, KeyError) as e:  # noqa: PERF203
                last = e
                if attempt == n or not getattr(self, "retry_on_failure", True):
                    break
                logging.warning("sample %s of %s failed (%s); retrying a random index", idx,
                                getattr(self, "repo_id", "?"), e)
                idx = random.randrange(len(self))
        raise last  # type: ignore[misc]

    return wrapped


class LeRobotDatasetMetadata(HubTransferMixin):
    def __init__(self, repo_id: str, root: str | Path | None = None, revision: str | None = None):
        self.repo_id = repo_id
        self.root = Path(root) if root is not None else HF_HOME / repo_id
        self.revision = revision
        if not (self.root / INFO_PATH).exists():
            # not on disk: the metadata folder alone is small, fetch it (the data follows per selected episode)
            try:
                self.root.mkdir(parents=True, exist_ok=True)
                self.pull_from_repo(allow_patterns="meta/")
            except Exception as exc:  # noqa: BLE001 - offline, unknown repository, no credentials: one message
                with contextlib.suppress(OSError):
                    self.root.rmdir()                   # leave no empty folder behind
                raise FileNotFoundError(
                    f"dataset {repo_id!r} not found under {self.root} and it could not be fetched from the hub "
                    f"({type(exc).__name__}: {exc}); place the dataset on disk and pass `root`") from exc
            if not (self.root / INFO_PATH).exists():
                raise FileNotFoundError(f"dataset {repo_id!r}: the hub repository has no {INFO_PATH}")
        self.load_metadata()

    def load_metadata(self) -> None:
        self.info = load_info(self.root)
        self.version = get_version(self.info)
        check_version_compatibility(self.repo_id, self.version)
        self.tasks, self.task_to_task_index = load_tasks(self.root, self.version)
        self.episodes = load_episodes(self.root, self.version)
        self.stats = load_stats(self.root, self.version)
        self.episodes_stats = load_episodes_stats(self.root) if self.version == "v2.1" else {}
        self.advantages: dict | None = None
        adv = self.root / "meta" / "advantages.json"
        if adv.exists():
            import json
            raw = json.loads(adv.read_text())
            self.advantages = {(int(k.split(",")[0]), float(k.split(",")[1])): float(v) for k, v in raw.items()}

    # -- simple views ---------------------------------------------------------------------------------
    @property
    def fps(self) -> int:
        return int(self.info["fps"])

    @property
    def features(self) -> dict[str, dict]:
        return self.info["features"]

    @property
    def robot_type(self) -> str | None:
        return self.info.get("robot_type")

    @property
    def control_mode(self) -> str | None:
        return self.info.get("control_mode")

    @property
    def image_keys(self) -> list[str]:
        return [k for k, ft in self.features.items() if ft["dtype"] == "image"]

    @property
    def video_keys(self) -> list[str]:
        return [k for k, ft in self.features.items() if ft["dtype"] == "video"]

    @property
    def camera_keys(self) -> list[str]:
        return [k for k, ft in self.features.items() if ft["dtype"] in ("image", "video")]

    @property
    def names(self) -> dict[str, Any]:
        return {k: ft.get("names") for k, ft in self.features.items()}

    @property
    def shapes(self) -> dict[str, tuple]:
        return {k: tuple(ft["shape"]) for k, ft in self.features.items()}

    @property
    def total_episodes(self) -> int:
        return int(self.info["total_episodes"])

    @property
    def total_frames(self) -> int:
        return int(self.info["total_frames"])

    @property
    def total_tasks(self) -> int:
        return int(self.info.get("total_tasks", len(self.tasks)))

    @property
    def chunks_size(self) -> int:
        return int(self.info.get("chunks_size", DEFAULT_CHUNK_SIZE))

    def get_episode_chunk(self, ep_index: int) -> int:
        return ep_index // self.chunks_size

    def get_data_file_path(self, ep_index: int) -> Path:
        if self.version == "v3.0":
            ep = self.episodes[ep_index]
            return Path(self.info["data_path"].format(chunk_index=ep["data/chunk_index"], file_index=ep["data/file_index"]))
        return Path(self.info.get("data_path", DEFAULT_PARQUET_PATH).format(
            episode_chunk=self.get_episode_chunk(ep_index), episode_index=ep_index))

    def get_video_file_path(self, ep_index: int, vid_key: str) -> Path:
        if self.version == "v3.0":
            ep = self.episodes[ep_index]
            return Path(self.info["video_path"].format(video_key=vid_key, chunk_index=ep[f"videos/{vid_key}/chunk_index"],
                                                       file_index=ep[f"videos/{vid_key}/file_index"]))
        return Path(self.info.get("video_path", DEFAULT_VIDEO_PATH).format(
            episode_chunk=self.get_episode_chunk(ep_index), video_key=vid_key, episode_index=ep_index))

    def video_time_offset(self, ep_index: int, vid_key: str) -> float:
        """v3.0 packs several episodes into one video file; the episode starts at this timestamp."""
        if self.version == "v3.0":
            return float(self.episodes[ep_index].get(f"videos/{vid_key}/from_timestamp", 0.0))
        return 0.0

    def get_task_index(self, task: str) -> int | None:
        return self.task_to_task_index.get(task)

    # -- writing (v2.1) ---------------------------------------------------------------------------------
    def add_task(self, task: str) -> int:
        if task in self.task_to_task_index:
            raise ValueError(f"The task '{task}' already exists and can't be added twice.")
        idx = self.info["total_tasks"]
        self.task_to_task_index[task] = idx
        self.tasks[idx] = task
        self.info["total_tasks"] += 1
        append_jsonlines({"task_index": idx, "task": task}, self.root / TASKS_PATH)
        return idx

    def save_episode(self, episode_index: int, length: int, tasks: list[str], stats: dict) -> None:
        self.info["total_episodes"] += 1
        self.info["total_frames"] += length
        chunk = self.get_episode_chunk(episode_index)
        if chunk >= self.info["total_chunks"]:
            self.info["total_chunks"] += 1
        self.info["splits"] = {"train": f"0:{self.info['total_episodes']}"}
        self.info["total_videos"] += len(self.video_keys)
        write_json(_jsonable_info(self.info), self.root / INFO_PATH)
        ep = {"episode_index": episode_index, "tasks": tasks, "length": length}
        self.episodes[episode_index] = ep
        append_jsonlines(ep, self.root / EPISODES_PATH)
        self.episodes_stats[episode_index] = stats
        self.stats = aggregate_stats([self.stats, stats]) if self.stats else stats
        append_jsonlines({"episode_index": episode_index, "stats": serialize_stats(stats)},
                         self.root / EPISODES_STATS_PATH)

    @classmethod
    def create(cls, repo_id: str, fps: int, root: str | Path | None = None, robot_type: str | None = None,
               features: dict | None = None, use_videos: bool = True) -> "LeRobotDatasetMetadata":
        obj = cls.__new__(cls)
        obj.repo_id = repo_id
        obj.root = Path(root) if root is not None else HF_HOME / repo_id
        obj.root.mkdir(parents=True, exist_ok=False)
        if features is None:
            raise ValueError("Dataset features must be provided explicitly.")
        feats = {k: dict(v) for k, v in {**features, **DEFAULT_FEATURES}.items()}
        for ft in feats.values():
            ft["shape"] = tuple(ft["shape"])
            if ft["dtype"] in ("image", "video"):
                ft["dtype"] = "video" if use_videos else "image"
        obj.info = {"codebase_version": CODEBASE_VERSION, "robot_type": robot_type, "total_episodes": 0,
                    "total_frames": 0, "total_tasks": 0, "total_videos": 0, "total_chunks": 0,
                    "chunks_size": DEFAULT_CHUNK_SIZE, "fps": fps, "splits": {}, "data_path": DEFAULT_PARQUET_PATH,
                    "video_path": DEFAULT_VIDEO_PATH if use_videos else None, "features": feats}
        obj.version = CODEBASE_VERSION
        obj.revision = None
        obj.tasks, obj.task_to_task_index, obj.episodes, obj.episodes_stats = {}, {}, {}, {}
        obj.stats, obj.advantages = None, None
        write_json(_jsonable_info(obj.info), obj.root / INFO_PATH)
        return obj


def _update_video_info(meta: "LeRobotDatasetMetadata", skip_keys: set[str] | None = None) -> None:
    """Fills the ``info`` block of every video feature (size, codec, pixel format, fps) from the FIRST episode's file,
    assuming all videos were encoded alike; keys in ``skip_keys`` and keys whose file does not exist yet are left."""
    from .video_utils import get_video_info
    for key in meta.video_keys:
        if skip_keys and key in skip_keys:
            continue
        if not meta.features[key].get("info"):
            path = meta.root / meta.get_video_file_path(0, key)
            if path.is_file():
                meta.info["features"][key]["info"] = get_video_info(path)


def _jsonable_info(info: dict) -> dict:
    out = dict(info)
    out["features"] = {k: {**ft, "shape": list(ft["shape"])} for k, ft in info["features"].items()}
    return out


def resolve_selected_episodes(all_episodes, episodes: list[int] | None, excluded_episodes: list[int] | None,
                              repo_id: str = "") -> list[int] | None:
    """``(episodes if given else all) - excluded``, sorted; the deny list wins over the allow list.  ``None`` means
    "no selection active: every episode".  A deny list that empties the selection is an error."""
    if not excluded_episodes:
        return sorted(episodes) if episodes is not None else None
    excluded = set(excluded_episodes)
    base = list(episodes) if episodes is not None else list(all_episodes)
    kept = sorted(e for e in base if e not in excluded)
    if not kept:
        raise ValueError(f"excluded_episodes removed every episode from {repo_id!r} (base={len(base)} episodes, "
                         f"excluded={sorted(excluded)}).")
    return kept


def aggregate_selected_stats(meta: "LeRobotDatasetMetadata", episodes: list[int] | None = None,
                             excluded_episodes: list[int] | None = None) -> dict:
    """Per-feature statistics over the SELECTED episodes (what the policy trains on), for off-line consumers such as
    the tokenizer fit and the normalisation diagnostic.  Falls back to the dataset-level statistics when no selection
    is active or the dataset has no per-episode statistics (v2.0)."""
    selected = resolve_selected_episodes(meta.episodes, episodes, excluded_episodes, meta.repo_id)
    if selected is None or not meta.episodes_stats:
        return meta.stats
    return aggregate_stats([meta.episodes_stats[e] for e in selected])


# ------------------------------------------------------------------------------------------------ base
class BaseDataset(torch.utils.data.Dataset):
    """Shared standard-format conversion (LeRobot and VQA datasets both end here)."""

    def __init__(self, cfg, *, name_map: dict[str, str] | None = None, train: bool = True):
        self.cfg = cfg
        self.resolution = tuple(cfg.resolution)
        self.num_cams = cfg.num_cams
        self.max_state_dim, self.max_action_dim = cfg.max_state_dim, cfg.max_action_dim
        self.action_chunk = cfg.action_chunk
        self.n_obs_history = cfg.dataset_mixture.n_obs_history
        # the two augmentation switches of a dataset instance: optional-key dropout rolls (masking / zero-fill; the
        # choice of WHICH future frame becomes a subgoal stays random either way) and per-task prompt substitution.
        # The validation subset is a shallow copy with its own values (shallow_copy_with_dropout).
        self.enable_optional_key_dropout = bool(train)
        self.enable_prompt_substitution = bool(train)
        self._name_map = name_map or {}
        self.state_index: list[int] | None = None
        self.action_index: list[int] | None = None
        self.delta_action_state_map: dict | None = None
        self._opt_rng = random.Random(0)

    @property
    def train(self) -> bool:
        return self.enable_optional_key_dropout

    @train.setter
    def train(self, flag: bool) -> None:
        self.enable_optional_key_dropout = bool(flag)

    def shallow_copy_with_dropout(self, *, enable_dropout: bool, enable_prompt_substitution: bool = False) -> "BaseDataset":
        """A copy that shares the table, metadata, index and cached segment tables by reference and differs only in the
        two augmentation switches: how the validation subset gets its own instance."""
        import copy
        clone = copy.copy(self)
        clone.enable_optional_key_dropout = enable_dropout
        clone.enable_prompt_substitution = enable_prompt_substitution
        return clone

    def _assert_image_in_unit_range(self, img: Tensor, *, name: str, expect_temporal: bool | None = None) -> None:
        """Rank (``(3, H, W)``, or ``(T, 3, H, W)`` with an observation history; subgoals pass ``expect_temporal=False``),
        three channels and values in [0, 1]."""
        if expect_temporal is None:
            expect_temporal = self.n_obs_history is not None
        ndim, cdim, desc = (4, 1, "(T, 3, H, W)") if expect_temporal else (3, 0, "(3, H, W)")
        ok = img.dim() == ndim and img.shape[cdim] == 3 and float(img.min()) >= -1e-6 and float(img.max()) <= 1.0 + 1e-6
        if not ok:
            raise AssertionError(f"Expected image {name} to have shape {desc} with values in [0, 1], got shape "
                                 f"{tuple(img.shape)}, min={float(img.min())}, max={float(img.max())}, "
                                 f"self={self._get_feature_mapping_key()}.")

    # hooks -------------------------------------------------------------------------------------------
    def _get_name_map(self) -> dict[str, str]:
        return self._name_map

    def _get_feature_mapping_key(self) -> str:
        return getattr(self, "repo_id", type(self).__name__)

    @staticmethod
    def pad_vector(v: Tensor, new_dim: int) -> Tensor:
        if v.shape[-1] == new_dim:
            return v
        if v.shape[-1] > new_dim:
            raise ValueError(f"vector of width {v.shape[-1]} does not fit into {new_dim}")
        out = v.new_zeros(*v.shape[:-1], new_dim)
        out[..., :v.shape[-1]] = v
        return out

    def _standardize_images(self, item: dict, out: dict, num_cams: int) -> list[bool]:
        name_map = self._get_name_map()
        H, W = self.resolution
        pads: list[bool] = []
        last = None
        for i in range(num_cams):
            raw = name_map.get(f"camera{i}")
            if raw is not None and raw in item:
                img = item[raw]
                img = img.float()
                if img.shape[-3] not in (1, 3) and img.shape[-1] in (1, 3):
                    img = img.movedim(-1, -3)
                lead = img.shape[:-3]
                flat = img.reshape(-1, *img.shape[-3:])
                if tuple(flat.shape[-2:]) != (H, W):
                    flat = ops.resize_with_pad(flat, W, H, pad_value=0.0)
                img = flat.reshape(*lead, *flat.shape[-3:])
                out[f"camera{i}"] = img
                last = img
                pads.append(False)
            else:
                shape = last.shape if last is not None else (
                    (self.n_obs_history, 3, H, W) if self.n_obs_history else (3, H, W))
                out[f"camera{i}"] = torch.zeros(shape)
                pads.append(True)
        return pads

    def _apply_column_index_and_delta(self, out: dict) -> None:
        who = getattr(self, "repo_id", None) or type(self).__name__
        out["state"] = apply_column_index(out["state"], self.state_index, what="state", who=who)
        out["actions"] = apply_column_index(out["actions"], self.action_index, what="action", who=who)
        if self.delta_action_state_map:      # post-index positions (resolved once in the constructor)
            out["actions"] = subtract_chunk_start_state(out["actions"], out["state"], self.delta_action_state_map)

    def _roll(self, p: float) -> bool:
        """True = drop.  Dropout rolls are active in training (or when validation opts in)."""
        if not self.enable_optional_key_dropout:
            return False
        return self._opt_rng.random() < p

    def _emit_optional_keys(self, item: dict, out: dict) -> None:
        """Memory / subgoal / metadata keys with their training-time dropout.  Every key is ALWAYS present: numeric and
        image keys are zero-filled with a parallel ``<key>_is_pad`` flag when absent or masked, string keys use the
        empty string as the pad signal.  Order of the rolls (all of them off when ``enable_optional_key_dropout`` is):

        1. ``history_state_drop_prob``: ``obs_history_is_pad`` all True and the historical camera frames zeroed; the
           state history is left alone here (zeroing a raw state before normalisation would turn 0 into -mean/std; the
           policy zeroes it after normalising) and the current step is always kept;
        2. subgoals are all-or-none: ``subgoal_is_pad`` is one flag for every ``subgoal{k}`` (their drop roll was taken
           before the frames were decoded, in ``_load_subgoal_frames``);
        3. ``response_drop_prob``: only when the subgoals were kept;
        4. ``metadata_drop_all_prob`` masks speed, mistake, quality, robot type and control mode together, otherwise
           ``metadata_drop_each_prob`` rolls per field.  ``fps`` (the mixture's ``action_freq`` when it resamples, else
           the dataset's own rate) takes part in no roll; a dataset without a frame rate emits ``fps=0`` padded."""
        mix = self.cfg.dataset_mixture
        if self._roll(mix.history_state_drop_prob):
            if self.n_obs_history is not None:
                out["obs_history_is_pad"] = torch.ones(self.n_obs_history, dtype=torch.bool)
                if self.n_obs_history > 1:
                    for k in range(self.num_cams):
                        if f"camera{k}" in out:
                            out[f"camera{k}"][:-1] = 0
            else:
                out["obs_history_is_pad"] = torch.tensor([True], dtype=torch.bool)

        H, W = self.resolution
        pad_subgoals = not all(item.get(f"subgoal{k}_raw") is not None for k in range(self.num_cams))
        for k in range(self.num_cams):
            if pad_subgoals:
                out[f"subgoal{k}"] = torch.zeros(3, H, W)
            else:
                im = item[f"subgoal{k}_raw"].float()
                if tuple(im.shape[-2:]) != (H, W):
                    im = ops.resize_with_pad(im[None], W, H, pad_value=0.0)[0]
                out[f"subgoal{k}"] = im
            self._assert_image_in_unit_range(out[f"subgoal{k}"], name=f"subgoal{k}", expect_temporal=False)
        out["subgoal_is_pad"] = torch.tensor(pad_subgoals)
        if not pad_subgoals and self._roll(mix.response_drop_prob):
            out["response"] = ""

        out["memory"] = item["memory_raw"] if isinstance(item.get("memory_raw"), str) else ""
        out["next_memory"] = item["next_memory_raw"] if isinstance(item.get("next_memory_raw"), str) else ""

        drop_all = self._roll(mix.metadata_drop_all_prob)
        for key, dtype in (("speed", torch.long), ("mistake", torch.bool), ("quality", torch.long)):
            raw = item.get(f"{key}_raw")
            dropped = drop_all or self._roll(mix.metadata_drop_each_prob)
            if raw is None or dropped:
                out[key] = torch.tensor(False if dtype is torch.bool else 0, dtype=dtype)
                out[f"{key}_is_pad"] = torch.tensor(True)
            else:
                out[key] = torch.tensor(bool(raw) if dtype is torch.bool else int(raw), dtype=dtype)
                out[f"{key}_is_pad"] = torch.tensor(False)
        for key in ("robot_type", "control_mode"):
            dropped = drop_all or self._roll(mix.metadata_drop_each_prob)
            out[key] = "" if dropped else str(item.get(key) or "")
        if mix.emit_fps:
            native = item.get("fps")
            if native is None:
                out["fps"], out["fps_is_pad"] = torch.tensor(0, dtype=torch.long), torch.tensor(True)
            else:
                eff = int(mix.action_freq) if getattr(mix, "action_freq", None) is not None else int(native)
                out["fps"], out["fps_is_pad"] = torch.tensor(eff, dtype=torch.long), torch.tensor(False)

    @staticmethod
    def _resolve_episode_success(item: dict, episodes_info: dict, name_map: dict[str, str],
                                 episode_stats: dict | None = None) -> bool | None:
        """The ``success`` role of the current sample, first hit wins: the column mapped to ``success`` read from the
        frame, then from the episode's metadata record; that column's per-episode ``mean`` thresholded at 0.5; the
        plain ``success`` key of the episode record.  ``None`` = unlabelled (not the same as "failed").  Pass only
        genuinely per-episode statistics (reference ``src/opentau/datasets/lerobot_dataset.py:2596-2650``)."""
        def first(v):
            return np.asarray(v.cpu() if isinstance(v, Tensor) else v).reshape(-1)[0]

        col = name_map.get("success")
        if col is not None:
            value = item.get(col)
            if value is None:
                value = episodes_info.get(col)
            if value is not None:
                return bool(first(value))
            stat = ((episode_stats or {}).get(col) or {}).get("mean")
            if stat is not None:
                return float(first(stat)) >= 0.5
        value = episodes_info.get("success")
        return None if value is None else bool(first(value))

    @staticmethod
    def _count_success_role_varying_episodes(episodes_stats, success_col: str) -> tuple[int, int]:
        """``(varying, checked)``: episodes whose mapped success column has min != max, among those that have both
        aggregates (0 checked = nothing provable)."""
        varying = checked = 0
        entries = episodes_stats.values() if isinstance(episodes_stats, dict) else episodes_stats
        for st in entries:
            col = (st or {}).get(success_col) or {}
            if col.get("min") is None or col.get("max") is None:
                continue
            checked += 1
            lo, hi = np.asarray(col["min"]).reshape(-1)[0], np.asarray(col["max"]).reshape(-1)[0]
            varying += int(lo != hi)
        return varying, checked

    def _attach_mistake_raw(self, item: dict, episodes_info: dict, ep_idx: int) -> bool | None:
        """``mistake_raw`` from the frame column mapped to ``mistake`` (segment-grained, wins), else the inverse of the
        resolved ``success`` role; neither -> no key.  Returns the resolved success for the return bins."""
        name_map = self._get_name_map()
        stats = None
        if getattr(self.meta, "version", "") != "v2.0":       # v2.0 has dataset-level statistics only
            stats = (getattr(self.meta, "episodes_stats", None) or {}).get(ep_idx)
        success = self._resolve_episode_success(item, episodes_info, name_map, stats)
        mistake_col = name_map.get("mistake", "mistake")
        if mistake_col in item:
            item["mistake_raw"] = bool(np.asarray(item[mistake_col].cpu() if isinstance(item[mistake_col], Tensor)
                                                  else item[mistake_col]).reshape(-1)[0])
        elif success is not None:
            item["mistake_raw"] = not success
        return success

    def _to_standard_data_format(self, item: dict) -> dict:
        name_map = self._get_name_map()
        out: dict[str, Any] = {}
        img_is_pad = self._standardize_images(item, out, self.num_cams)
        for new_key, key in name_map.items():
            if "camera" in new_key or new_key in ("mistake", "success") or key not in item:
                continue
            out[new_key] = item[key]
        out.setdefault("response", "")
        self._apply_column_index_and_delta(out)
        real_action_dim = int(out["actions"].shape[-1])
        if not 0 < real_action_dim <= self.max_action_dim:
            raise ValueError(f"real action dim {real_action_dim} is outside (0, {self.max_action_dim}] "
                             f"(dataset={getattr(self, 'repo_id', '?')})")
        out["real_action_dim"] = torch.tensor(real_action_dim, dtype=torch.long)
        out["state"] = self.pad_vector(out["state"].float(), self.max_state_dim)
        out["actions"] = self.pad_vector(out["actions"].float(), self.max_action_dim)
        out["img_is_pad"] = torch.tensor(img_is_pad, dtype=torch.bool)
        a_key = name_map.get("actions", "actions")
        out["action_is_pad"] = item.get(f"{a_key}_is_pad", torch.zeros(out["actions"].shape[0], dtype=torch.bool))
        s_pad = item.get(f"{name_map.get('state', 'state')}_is_pad")
        if s_pad is not None:
            out["obs_history_is_pad"] = s_pad
        elif self.n_obs_history is not None:
            out["obs_history_is_pad"] = torch.zeros(self.n_obs_history, dtype=torch.bool)
        else:
            out["obs_history_is_pad"] = torch.tensor([False], dtype=torch.bool)
        self._emit_optional_keys(item, out)
        for k, v in out.items():
            if isinstance(v, Tensor) and v.dtype.is_floating_point:
                out[k] = v.to(torch.bfloat16)
        out["source"] = self._get_feature_mapping_key()
        for k in ("episode_index", "frame_index"):
            v = item.get(k)
            out[k] = int(v.item() if torch.is_tensor(v) else v) if v is not None else -1
        return out


# ------------------------------------------------------------------------------------------------ reader
class LeRobotDataset(BaseDataset, HubTransferMixin):
    def __init__(self, cfg, repo_id: str, root: str | Path | None = None, episodes: list[int] | None = None,
                 image_transforms: Callable | None = None, delta_timestamps: dict[str, list[float]] | None = None,
                 tolerance_s: float = 1e-4, revision: str | None = None, video_backend: str | None = None,
                 image_resample_strategy: str = "nearest", vector_resample_strategy: str = "nearest",
                 standardize: bool = True, dataset_cfg=None, train: bool = True, meta: LeRobotDatasetMetadata | None = None,
                 return_advantage_input: bool = False, excluded_episodes: list[int] | None = None):
        self.repo_id = repo_id
        self.meta = meta or LeRobotDatasetMetadata(repo_id, root, revision)
        self.root = self.meta.root
        dcfg = dataset_cfg
        name_map = get_mapping(repo_id, self.meta.features, getattr(dcfg, "data_features_name_mapping", None),
                               control_mode=(getattr(dcfg, "control_mode", None) or self.meta.control_mode))
        super().__init__(cfg, name_map=name_map, train=train)
        if excluded_episodes is None and dcfg is not None:
            excluded_episodes = getattr(dcfg, "excluded_episodes", None)
        selected = resolve_selected_episodes(self.meta.episodes, episodes, excluded_episodes, repo_id)
        if selected is not None and self.meta.episodes_stats:
            # the mixture normaliser pools ``meta.stats``: it must describe the episodes that are trained on, not the
            # whole dataset on disk (a v2.0 dataset has no per-episode statistics and keeps the dataset-level ones)
            # (on a shallow copy: a metadata object handed in by the caller may be shared with the other split)
            import copy
            self.meta = copy.copy(self.meta)
            self.meta.stats = aggregate_stats([self.meta.episodes_stats[e] for e in selected])
        self.episodes = selected if selected is not None else sorted(self.meta.episodes)
        self.revision = revision if revision is not None else self.meta.revision
        self._episodes_were_specified = selected is not None
        self._fetch_missing_files()
        self.image_transforms = image_transforms
        self.delta_timestamps = {k: np.asarray(v, dtype=np.float64) for k, v in (delta_timestamps or {}).items()}
        self.tolerance_s = tolerance_s
        self.video_backend = video_backend
        if image_resample_strategy not in ("nearest", "linear") or vector_resample_strategy not in ("nearest", "linear"):
            raise ValueError("resample strategies must be 'nearest' or 'linear'")
        self.image_resample_strategy, self.vector_resample_strategy = image_resample_strategy, vector_resample_strategy
        self.standardize = standardize
        self.return_advantage_input = return_advantage_input
        self.retry_on_failure = True
        if dcfg is not None:
            self.state_index, self.action_index = dcfg.state_index, dcfg.action_index
            if dcfg.use_delta_joint_actions:
                # the config's map is written against the stored columns; what is applied (and published to the
                # policy through the mixture metadata) is its image after the column selection
                shape = (self.meta.features.get(self._name_map.get("actions", "action"), {}) or {}).get("shape")
                width = len(dcfg.action_index) if dcfg.action_index is not None else (shape[-1] if shape else None)
                self.delta_action_state_map = resolve_delta_map(dcfg.delta_action_state_map, dcfg.action_index,
                                                                dcfg.state_index, who=repo_id, action_dim=width)
            self.prompt_substitutions = dcfg.prompt_substitutions
            self.robot_type = dcfg.robot_type if dcfg.robot_type is not None else self.meta.robot_type
            self.control_mode = dcfg.control_mode if dcfg.control_mode is not None else self.meta.control_mode
        else:
            self.prompt_substitutions, self.robot_type, self.control_mode = None, self.meta.robot_type, self.meta.control_mode
        self._load_table()
        self.episode_data_index = get_episode_data_index(self.meta.episodes, self.episodes)
        if "timestamp" in self._numeric:
            check_timestamps_sync(self._numeric["timestamp"].numpy(), self._numeric["episode_index"].numpy(),
                                  {"to": np.asarray(self.episode_data_index["to"])}, self.fps, self.tolerance_s)
        self.epi2idx = {ep: i for i, ep in enumerate(self.episodes)}
        self._build_episode_tables()

    def _build_episode_tables(self) -> None:
        """Per-episode caches of the optional-key path, read once: lengths, segment start frames (a legacy episode is
        one segment starting at 0), the speed label of every selected episode, one memory string per segment."""
        from .speed_percentiles import (episode_to_task_index, load_or_compute_speed_percentiles,
                                        speed_bucket_by_episode)
        self.episode_lengths = {ep: int(info["length"]) for ep, info in self.meta.episodes.items()}
        self.segment_starts_by_episode: dict[int, np.ndarray] = {}
        for ep, info in self.meta.episodes.items():
            starts = info.get("segments")
            if starts is None or len(starts) == 0:
                starts = [0]
            # a list of start frames; [start, end) pairs are accepted and reduced to their starts
            starts = [int(s[0]) if isinstance(s, (list, tuple)) else int(s) for s in starts]
            self.segment_starts_by_episode[ep] = np.asarray(starts, dtype=np.int64)
        first_rows = {ep: int(self._numeric["task_index"][int(self.episode_data_index["from"][self.epi2idx[ep]])])
                      for ep in self.episodes} if "task_index" in self._numeric else {}
        self.episode_to_task_index = episode_to_task_index(first_rows, set(self.meta.task_to_task_index.values()))
        if any("speed" in self.meta.episodes[ep] for ep in self.episodes):
            # an explicit per-episode label in the metadata wins over the length ranking
            self.speed_percentiles_by_task = {}
            self.speed_raw_by_episode = {ep: int(self.meta.episodes[ep].get("speed", 0) or 0) for ep in self.episodes}
        else:
            self.speed_percentiles_by_task = load_or_compute_speed_percentiles(
                self.root, self.episode_lengths, self.episode_to_task_index, self.meta.task_to_task_index)
            self.speed_raw_by_episode = speed_bucket_by_episode(self.episodes, self.episode_lengths,
                                                                self.episode_to_task_index,
                                                                self.speed_percentiles_by_task)
        self.segment_memories_by_episode: dict[int, list[str]] = {}
        has_memory = "memory" in self._string_cols
        col = self._table.column("memory") if has_memory else None
        for ep in self.episodes:
            starts = self.segment_starts_by_episode[ep]
            if has_memory:
                ep_start = int(self.episode_data_index["from"][self.epi2idx[ep]])
                self.segment_memories_by_episode[ep] = [str(col[ep_start + int(s)].as_py() or "") for s in starts]
            else:
                self.segment_memories_by_episode[ep] = [""] * len(starts)

    # -- segments, memory, subgoals -----------------------------------------------------------------------
    def _lookup_segment_index(self, ep_idx: int, frame_in_ep: int) -> int:
        starts = self.segment_starts_by_episode[ep_idx]
        return max(int(np.searchsorted(starts, frame_in_ep, side="right")) - 1, 0)

    def _segment_end_in_ep(self, ep_idx: int, seg_idx: int) -> int:
        """Exclusive end frame of a segment inside its episode."""
        starts = self.segment_starts_by_episode[ep_idx]
        return int(starts[seg_idx + 1]) if seg_idx + 1 < len(starts) else self.episode_lengths[ep_idx]

    def _lookup_next_memory(self, ep_idx: int, frame_in_ep: int) -> str:
        """The memory string that holds at frame ``frame_in_ep + 1`` (clipped at the episode's end)."""
        nxt = min(frame_in_ep + 1, self.episode_lengths[ep_idx] - 1)
        memories = self.segment_memories_by_episode.get(ep_idx, [""])
        if not memories:
            return ""
        return memories[min(self._lookup_segment_index(ep_idx, nxt), len(memories) - 1)]

    def _sample_subgoal_frame(self, ep_idx: int, frame_in_ep: int, *, at_end_of_segment: bool) -> int:
        """A future frame of the episode to serve as the subgoal: the last frame of the current segment, or one drawn
        uniformly from ``[t, t + 4 s]`` clipped to the segment and the episode.  Episodes without a ``segments``
        annotation get a fixed 4 s look-ahead (clipped to the episode), so legacy datasets still get supervision."""
        n = self.episode_lengths[ep_idx]
        window = int(round(4.0 * self.fps))
        if "segments" not in self.meta.episodes[ep_idx]:
            return min(frame_in_ep + window, n - 1)
        seg = self._lookup_segment_index(ep_idx, frame_in_ep)
        upper = max(min(self._segment_end_in_ep(ep_idx, seg), n) - 1, frame_in_ep)
        if at_end_of_segment:
            return upper
        top = min(frame_in_ep + window, upper)
        return frame_in_ep if top <= frame_in_ep else self._opt_rng.randint(frame_in_ep, top)

    def _fetch_missing_files(self) -> None:
        """Data (and video) files of the selected episodes that are not under the root are fetched from the hub; a
        complete root makes no request at all."""
        files = self.get_episodes_file_paths()
        missing = [f for f in dict.fromkeys(files) if not (self.root / f).is_file()]
        if not missing:
            return
        try:
            self.download_episodes(download_videos=True)
        except Exception as exc:  # noqa: BLE001
            raise FileNotFoundError(f"dataset {self.repo_id!r}: {len(missing)} file(s) of the selected episodes are not "
                                    f"under {self.root} (first: {missing[0]}) and could not be fetched from the hub "
                                    f"({type(exc).__name__}: {exc})") from exc

    # -- table ------------------------------------------------------------------------------------------
    def _load_table(self) -> None:
        import pyarrow as pa
        import pyarrow.parquet as pq
        files: list[Path] = []
        for ep in self.episodes:
            f = self.root / self.meta.get_data_file_path(ep)
            if f not in files:
                files.append(f)
        tables = [pq.read_table(f) for f in files]
        table = pa.concat_tables(tables, promote_options="default") if len(tables) > 1 else tables[0]
        ep_col = np.asarray(table.column("episode_index").to_numpy())
        keep = np.isin(ep_col, np.asarray(self.episodes))
        if not keep.all():
            table = table.filter(pa.array(keep))
        order = np.lexsort((np.asarray(table.column("frame_index").to_numpy()),
                            np.asarray(table.column("episode_index").to_numpy())))
        if not (order == np.arange(len(order))).all():
            table = table.take(pa.array(order))
        self._table = table
        self._numeric: dict[str, Tensor] = {}
        self._image_cols: list[str] = []
        self._string_cols: list[str] = []
        for name in table.column_names:
            ft = self.meta.features.get(name)
            if ft is not None and ft["dtype"] == "image":
                self._image_cols.append(name)
                continue
            if ft is not None and ft["dtype"] == "string" or pa.types.is_string(table.schema.field(name).type):
                self._string_cols.append(name)
                continue
            col = table.column(name).to_numpy(zero_copy_only=False)
            if col.dtype == object:
                col = np.stack([np.asarray(x) for x in col])
            self._numeric[name] = torch.from_numpy(np.ascontiguousarray(col))

    def __len__(self) -> int:
        return self._table.num_rows

    @property
    def num_frames(self) -> int:
        return len(self)

    @property
    def num_episodes(self) -> int:
        return len(self.episodes)

    @property
    def fps(self) -> int:
        return self.meta.fps

    @property
    def features(self) -> dict[str, dict]:
        return self.meta.features

    # -- queries ----------------------------------------------------------------------------------------
    def _soft_indices(self, idx: int, ep_idx: int) -> tuple[dict[str, np.ndarray], dict[str, Tensor]]:
        i = self.epi2idx[ep_idx]
        ep_start, ep_end = int(self.episode_data_index["from"][i]), int(self.episode_data_index["to"][i])
        q, pad = {}, {}
        for key, dts in self.delta_timestamps.items():
            d = dts * self.fps
            q[key] = np.clip(idx + d, ep_start, ep_end - 1)
            pad[f"{key}_is_pad"] = torch.from_numpy((idx + d < ep_start - 1e-9) | (idx + d > ep_end - 1 + 1e-9))
        return q, pad

    def _query_vectors(self, soft: dict[str, np.ndarray]) -> dict[str, Tensor]:
        out = {}
        for key, s in soft.items():
            if key not in self._numeric:
                continue
            col = self._numeric[key]
            if self.vector_resample_strategy == "nearest" or not col.dtype.is_floating_point:
                out[key] = col[torch.from_numpy(np.round(s).astype(np.int64))]
            else:
                lo = np.floor(s).astype(np.int64)
                hi = np.minimum(lo + 1, len(col) - 1)
                w = torch.from_numpy(s - lo).to(col.dtype)
                while w.dim() < col[lo].dim():
                    w = w.unsqueeze(-1)
                out[key] = col[torch.from_numpy(lo)] * (1 - w) + col[torch.from_numpy(hi)] * w
        return out

    def _decode_image_cell(self, cell) -> Tensor:
        from PIL import Image
        if isinstance(cell, dict):
            raw = cell.get("bytes")
            img = Image.open(io.BytesIO(raw)) if raw is not None else Image.open(self.root / cell["path"])
        else:
            img = Image.open(io.BytesIO(cell))
        arr = np.asarray(img.convert("RGB"))
        return torch.from_numpy(arr).permute(2, 0, 1).float() / 255.0

    def _query_images(self, idx: int, soft: dict[str, np.ndarray]) -> dict[str, Tensor]:
        out = {}
        for key in self._image_cols:
            rows = np.round(soft[key]).astype(np.int64).tolist() if key in soft else [idx]
            col = self._table.column(key)
            out[key] = torch.stack([self._decode_image_cell(col[r].as_py()) for r in rows])
            if key not in soft:
                out[key] = out[key][0]
        return out

    def _query_videos(self, idx: int, ep_idx: int, soft: dict[str, np.ndarray]) -> dict[str, Tensor]:
        out = {}
        ep_start = int(self.episode_data_index["from"][self.epi2idx[ep_idx]])
        for key in self.meta.video_keys:
            if key in soft:
                ts = (np.round(soft[key]) if self.image_resample_strategy == "nearest" else soft[key]) - ep_start
                ts = (ts / self.fps).tolist()
            else:
                ts = [float(self._numeric["timestamp"][idx])]
            off = self.meta.video_time_offset(ep_idx, key)
            frames = decode_video_frames(self.root / self.meta.get_video_file_path(ep_idx, key),
                                         [t + off for t in ts], max(self.tolerance_s, 0.5 / self.fps), self.video_backend,
                                         fps=float(self.fps))
            out[key] = frames if key in soft else frames[0]
        return out

    def _resolve_task(self, task_index: int) -> str:
        task = self.meta.tasks.get(int(task_index), "")
        subs = self.prompt_substitutions
        if subs and self.enable_prompt_substitution and task in subs:
            return self._opt_rng.choice(subs[task])
        return task

    def _load_subgoal_frames(self, ep_idx: int, frame_in_ep: int) -> dict[str, Tensor]:
        """One goal frame per camera slot, for any dataset that has cameras.  The drop roll comes first, so a dropped
        subgoal costs no decode (with dropout switched off it is never rolled); the end-of-segment versus uniform roll
        happens once per sample and is shared by the cameras; video features are decoded at the frame's timestamp,
        image features come from the parquet row of the same frame."""
        if self.num_cams <= 0 or not self.meta.camera_keys:
            return {}
        mix = self.cfg.dataset_mixture
        if self.enable_optional_key_dropout and self._opt_rng.random() < mix.subgoal_drop_prob:
            return {}
        at_end = self._opt_rng.random() < mix.subgoal_end_of_segment_prob
        goal = self._sample_subgoal_frame(ep_idx, frame_in_ep, at_end_of_segment=at_end)
        gidx = int(self.episode_data_index["from"][self.epi2idx[ep_idx]]) + goal
        imgs = {**self._query_images(gidx, {}), **(self._query_videos(gidx, ep_idx, {}) if self.meta.video_keys else {})}
        out = {}
        for i in range(self.num_cams):
            raw = self._name_map.get(f"camera{i}")
            if raw in imgs:
                out[f"subgoal{i}_raw"] = imgs[raw]
        return out

    @retry_random_on_failure
    def __getitem__(self, idx: int) -> dict:
        idx = int(idx)
        if not 0 <= idx < len(self):
            raise IndexError(idx)
        item: dict[str, Any] = {k: v[idx] for k, v in self._numeric.items()}
        for k in self._string_cols:
            item[k] = self._table.column(k)[idx].as_py() or ""     # files without the column contribute nulls
        ep_idx = int(item["episode_index"])
        soft, padding = self._soft_indices(idx, ep_idx) if self.delta_timestamps else ({}, {})
        item.update(padding)
        item.update(self._query_vectors(soft))
        item.update(self._query_images(idx, soft))
        if self.meta.video_keys:
            item.update(self._query_videos(idx, ep_idx, soft))
        if self.image_transforms is not None:
            for cam in self.meta.camera_keys:
                if cam in item:
                    item[cam] = self.image_transforms(item[cam])
        item["task"] = self._resolve_task(int(item["task_index"]))
        for key, dts in self.delta_timestamps.items():
            if len(dts) == 1 and key in item and isinstance(item[key], Tensor):
                item[key] = item[key].squeeze(0)
        if not self.standardize:
            return item
        i = self.epi2idx[ep_idx]
        ep_start, ep_end = int(self.episode_data_index["from"][i]), int(self.episode_data_index["to"][i])
        frame_in_ep = idx - ep_start
        item["frame_index"] = frame_in_ep
        ep_info = self.meta.episodes[ep_idx]
        item.setdefault("response", "")
        if "memory" in item:
            item["memory_raw"] = str(item["memory"])
            item["next_memory_raw"] = self._lookup_next_memory(ep_idx, frame_in_ep)
        success = self._attach_mistake_raw(item, ep_info, ep_idx)
        if ep_info.get("quality") is not None:
            item["quality_raw"] = int(ep_info["quality"])
        item["speed_raw"] = self.speed_raw_by_episode.get(ep_idx)
        item["robot_type"], item["control_mode"], item["fps"] = self.robot_type, self.control_mode, self.fps
        item.update(self._load_subgoal_frames(ep_idx, frame_in_ep))
        timestamp = float(item["timestamp"])
        out = self._to_standard_data_format(item)
        adv = 0.0 if self.meta.advantages is None else self.meta.advantages.get((ep_idx, timestamp), 0.0)
        out["advantage"] = torch.tensor(adv, dtype=torch.bfloat16)
        success = True if success is None else bool(success)
        policy = getattr(self.cfg, "policy", None)
        rc = getattr(policy, "reward_config", None)
        if rc is not None and getattr(policy, "type", "") == "value":
            from ..policies.value.reward import calculate_return_bins_with_equal_width
            b, r = calculate_return_bins_with_equal_width(success, rc.number_of_bins, ep_end, rc.reward_normalizer, idx,
                                                          rc.C_neg)
            out["return_bin_idx"] = torch.tensor(b, dtype=torch.long)
            out["return_continuous"] = torch.tensor(r, dtype=torch.float32)
            if self.return_advantage_input:              # what the advantage tool needs to form n-step returns
                out.update(success=success, episode_end_idx=ep_end, current_idx=idx,
                           last_step=idx + rc.N_steps_look_ahead >= ep_end, episode_index=ep_idx, timestamp=timestamp)
        else:
            out["return_bin_idx"] = torch.tensor(0, dtype=torch.long)
            out["return_continuous"] = torch.tensor(0, dtype=torch.float32)
        if out["actions"].shape[0] != self.action_chunk or out["action_is_pad"].shape[0] != self.action_chunk:
            raise ValueError(f"action chunk of {out['actions'].shape[0]} steps, expected {self.action_chunk}")
        return out

    # -- recording API (v2.1) ---------------------------------------------------------------------------
    @classmethod
    def create(cls, repo_id: str, fps: int, root: str | Path | None = None, robot_type: str | None = None,
               features: dict | None = None, use_videos: bool = False, image_writer_threads: int = 0,
               deferred_video_keys: set[str] | list[str] | None = None, image_writer_processes: int = 0,
               tolerance_s: float = 1e-4) -> "LeRobotRecorder":
        """``deferred_video_keys``: video features whose frames are NOT handed to ``add_frame``; their files are
        attached after ``save_episode`` from recordings made elsewhere (``LeRobotRecorder.attach_video``)."""
        meta = LeRobotDatasetMetadata.create(repo_id, fps, root, robot_type, features, use_videos)
        return LeRobotRecorder(meta, image_writer_threads, deferred_video_keys, tolerance_s, image_writer_processes)


class LeRobotRecorder:
    """Frame-by-frame recording into the v2.1 layout: ``add_frame`` buffers, ``save_episode`` writes the parquet file,
    images or encoded videos, per-episode stats and the metadata records."""

    def __init__(self, meta: LeRobotDatasetMetadata, image_writer_threads: int = 0,
                 deferred_video_keys: set[str] | list[str] | None = None, tolerance_s: float = 1e-4,
                 image_writer_processes: int = 0):
        self.meta, self.root, self.fps = meta, meta.root, meta.fps
        self.features = meta.features
        self.tolerance_s = tolerance_s
        self.deferred_video_keys = set(deferred_video_keys or ())
        unknown = self.deferred_video_keys - set(meta.video_keys)
        if unknown:
            raise ValueError(f"deferred_video_keys {sorted(unknown)} are not video features ({meta.video_keys})")
        self.image_writer = None
        if image_writer_threads > 0 or image_writer_processes > 0:
            from .image_writer import AsyncImageWriter
            self.image_writer = AsyncImageWriter(num_processes=image_writer_processes,
                                                 num_threads=max(1, image_writer_threads))
        self.episode_buffer = self.create_episode_buffer()

    def create_episode_buffer(self, episode_index: int | None = None) -> dict:
        idx = self.meta.total_episodes if episode_index is None else episode_index
        return {**{k: [] for k in self.features}, "size": 0, "task": [], "episode_index": idx}

    def _image_path(self, key: str, ep: int, frame: int) -> Path:
        return self.root / DEFAULT_IMAGE_PATH.format(image_key=key, episode_index=ep, frame_index=frame)

    def add_frame(self, frame: dict) -> None:
        frame = {k: (v.numpy() if isinstance(v, Tensor) else v) for k, v in frame.items()}
        given = self.deferred_video_keys & set(frame)
        if given:
            raise ValueError(f"{sorted(given)} are deferred video keys: their frames come from attach_video, not add_frame")
        validate_frame(frame, {k: v for k, v in self.features.items() if k not in self.deferred_video_keys})
        buf = self.episode_buffer
        fi = buf["size"]
        buf["frame_index"].append(fi)
        buf["timestamp"].append(frame.pop("timestamp", fi / self.fps))
        buf["task"].append(frame.pop("task"))
        for k, v in frame.items():
            if self.features[k]["dtype"] in ("image", "video"):
                path = self._image_path(k, buf["episode_index"], fi)
                if self.image_writer is not None:
                    self.image_writer.save_image(v, path)
                else:
                    from .image_writer import write_image
                    write_image(np.asarray(v), path)
                buf[k].append(str(path))
            else:
                buf[k].append(np.asarray(v))
        buf["size"] += 1

    def save_episode(self) -> None:
        import pyarrow as pa
        import pyarrow.parquet as pq
        buf = self.episode_buffer
        validate_episode_buffer(buf, self.meta.total_episodes, self.features, self.deferred_video_keys)
        n, ep = buf["size"], buf["episode_index"]
        # frames 1 / fps apart: a recorder that dropped frames would shift every "k steps ahead" lookup
        check_timestamps_sync(np.asarray(buf["timestamp"], np.float64), np.full(n, ep), {"to": np.array([n])},
                              self.fps, self.tolerance_s)
        tasks = buf["task"]
        for t in dict.fromkeys(tasks):
            if self.meta.get_task_index(t) is None:
                self.meta.add_task(t)
        if self.image_writer is not None:
            self.image_writer.wait_until_done()
        cols: dict[str, Any] = {}
        stats_in: dict[str, np.ndarray] = {}
        start = self.meta.total_frames
        for k, ft in self.features.items():
            if k == "index":
                arr = np.arange(start, start + n)
            elif k == "episode_index":
                arr = np.full(n, ep)
            elif k == "task_index":
                arr = np.asarray([self.meta.get_task_index(t) for t in tasks])
            elif k in self.deferred_video_keys:
                continue                                   # no frames here: attached later, no statistics yet
            elif ft["dtype"] in ("image", "video"):
                paths = buf[k]
                from PIL import Image
                sel = sample_indices(n)
                stats_in[k] = np.stack([np.asarray(Image.open(paths[i]).convert("RGB"), dtype=np.float32).transpose(2, 0, 1) / 255.0
                                        for i in sel])
                if ft["dtype"] == "image":
                    cols[k] = pa.array([{"bytes": Path(p).read_bytes(), "path": None} for p in paths],
                                       type=pa.struct([("bytes", pa.binary()), ("path", pa.string())]))
                continue
            elif ft["dtype"] == "string":
                cols[k] = pa.array([str(x) for x in buf[k]])
                continue
            else:
                arr = np.stack(buf[k]) if len(buf[k]) else np.zeros((0,))
            arr = np.asarray(arr).astype(ft["dtype"])
            stats_in[k] = arr
            cols[k] = pa.array(arr.tolist() if arr.ndim > 1 else arr)
        path = self.root / self.meta.get_data_file_path(ep)
        path.parent.mkdir(parents=True, exist_ok=True)
        pq.write_table(pa.table(cols), path)
        self.encode_episode_videos(ep, skip_keys=self.deferred_video_keys)
        stats = compute_episode_stats(stats_in, {k: v for k, v in self.features.items() if k in stats_in})
        self.meta.save_episode(ep, n, list(dict.fromkeys(tasks)), stats)
        img_dir = self.root / "images"
        if img_dir.exists():
            shutil.rmtree(img_dir)
        self.episode_buffer = self.create_episode_buffer()

    # -- videos -----------------------------------------------------------------------------------------------
    def encode_episode_videos(self, episode_index: int, skip_keys: set[str] | None = None) -> dict[str, str]:
        """Frames written as image files -> one mp4 per video feature; a file that already exists is kept (resuming a
        recording).  Returns ``{video key: path}``."""
        out = {}
        for k in self.meta.video_keys:
            if skip_keys and k in skip_keys:
                continue
            path = self.root / self.meta.get_video_file_path(episode_index, k)
            out[k] = str(path)
            if not path.is_file():
                encode_video_frames(self._image_path(k, episode_index, 0).parent, path, self.fps, overwrite=True)
        return out

    def encode_videos(self) -> None:
        for ep in range(self.meta.total_episodes):
            self.encode_episode_videos(ep, skip_keys=self.deferred_video_keys)

    def attach_video(self, episode_index: int, video_key: str, input_video_path: str | Path, overwrite: bool = False,
                     start_time: float | None = None, **encode_kw) -> Path:
        """Attaches a recording made elsewhere to a saved episode: the source is resampled to the dataset's fps and
        trimmed to exactly the episode's number of frames (``start_time`` skips into the source) and lands at the
        standard video path.  Call ``update_video_info`` once all deferred videos are in place."""
        from .video_utils import resample_and_trim_video
        if video_key not in self.meta.video_keys:
            raise ValueError(f"'{video_key}' is not a video feature. Available video keys: {self.meta.video_keys}")
        if episode_index not in self.meta.episodes:
            raise ValueError(f"Episode {episode_index} does not exist. Total episodes: {self.meta.total_episodes}")
        if not Path(input_video_path).is_file():
            raise FileNotFoundError(input_video_path)
        out = self.root / self.meta.get_video_file_path(episode_index, video_key)
        if out.is_file() and not overwrite:
            logging.info("video already exists at %s, skipping (use overwrite=True to replace)", out)
            return out
        n = int(self.meta.episodes[episode_index]["length"])
        resample_and_trim_video(input_video_path, out, self.fps, n, overwrite=overwrite, start_time=start_time, **encode_kw)
        logging.info("attached video for episode %d, key '%s': %s -> %s (%d frames @ %d fps)", episode_index, video_key,
                     input_video_path, out, n, self.fps)
        return out

    def update_video_info(self) -> None:
        """Writes the real video properties (from the first episode's files) into ``meta/info.json``."""
        _update_video_info(self.meta)
        write_json(_jsonable_info(self.meta.info), self.root / INFO_PATH)

    def clear_episode_buffer(self) -> None:
        img_dir = self.root / "images"
        if img_dir.exists():
            shutil.rmtree(img_dir)
        self.episode_buffer = self.create_episode_buffer()

    def stop_image_writer(self) -> None:
        if self.image_writer is not None:
            self.image_writer.stop()
            self.image_writer = None
