"""On-disk LeRobot layout helpers: metadata IO, version checks, feature <-> policy-feature conversion.

Covers what the reader/writer need from the reference's ``src/opentau/datasets/utils.py:60-1704``: JSON / JSONL /
parquet metadata files of codebase versions v2.0, v2.1 and v3.0, path templates, the feature dictionary, and
``dataset_to_policy_features``.
"""

from __future__ import annotations

import json
from itertools import accumulate
from pathlib import Path
from typing import Any, Iterator

import numpy as np
import torch

from ..configs.types import FeatureType, PolicyFeature

INFO_PATH = "meta/info.json"
EPISODES_PATH = "meta/episodes.jsonl"
STATS_PATH = "meta/stats.json"
EPISODES_STATS_PATH = "meta/episodes_stats.jsonl"
TASKS_PATH = "meta/tasks.jsonl"
V30_EPISODES_DIR = "meta/episodes"
V30_TASKS_PATH = "meta/tasks.parquet"
DEFAULT_CHUNK_SIZE = 1000
DEFAULT_PARQUET_PATH = "data/chunk-{episode_chunk:03d}/episode_{episode_index:06d}.parquet"
DEFAULT_VIDEO_PATH = "videos/chunk-{episode_chunk:03d}/{video_key}/episode_{episode_index:06d}.mp4"
DEFAULT_IMAGE_PATH = "images/{image_key}/episode_{episode_index:06d}/frame_{frame_index:06d}.png"
CODEBASE_VERSION = "v2.1"
SUPPORTED_VERSIONS = ("v2.0", "v2.1", "v3.0")

DEFAULT_FEATURES = {
    "timestamp": {"dtype": "float32", "shape": (1,), "names": None},
    "frame_index": {"dtype": "int64", "shape": (1,), "names": None},
    "episode_index": {"dtype": "int64", "shape": (1,), "names": None},
    "index": {"dtype": "int64", "shape": (1,), "names": None},
    "task_index": {"dtype": "int64", "shape": (1,), "names": None},
}


class BackwardCompatibilityError(Exception):
    pass


def load_json(path: Path) -> Any:
    with open(path) as f:
        return json.load(f)


def write_json(data: Any, path: Path) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "w") as f:
        json.dump(data, f, indent=4, ensure_ascii=False)


def load_jsonlines(path: Path) -> list[Any]:
    with open(path) as f:
        return [json.loads(line) for line in f if line.strip()]


def write_jsonlines(rows: list[Any], path: Path) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "w") as f:
        for r in rows:
            f.write(json.dumps(r, ensure_ascii=False) + "\n")


def append_jsonlines(row: Any, path: Path) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "a") as f:
        f.write(json.dumps(row, ensure_ascii=False) + "\n")


def flatten_dict(d: dict, parent: str = "", sep: str = "/") -> dict:
    out = {}
    for k, v in d.items():
        key = f"{parent}{sep}{k}" if parent else k
        if isinstance(v, dict):
            out.update(flatten_dict(v, key, sep))
        else:
            out[key] = v
    return out


def unflatten_dict(d: dict, sep: str = "/") -> dict:
    out: dict = {}
    for k, v in d.items():
        cur = out
        parts = k.split(sep)
        for p in parts[:-1]:
            cur = cur.setdefault(p, {})
        cur[parts[-1]] = v
    return out


def serialize_stats(stats: dict) -> dict:
    return {k: {s: np.asarray(v).tolist() for s, v in d.items()} for k, d in stats.items()}


def cast_stats_to_numpy(stats: dict) -> dict:
    return {k: {s: np.asarray(v) for s, v in d.items()} for k, d in stats.items()}


def get_version(info: dict) -> str:
    v = str(info.get("codebase_version", "v2.0"))
    return v if v.startswith("v") else f"v{v}"


def check_version_compatibility(repo_id: str, version: str) -> None:
    if version not in SUPPORTED_VERSIONS:
        raise BackwardCompatibilityError(
            f"dataset {repo_id!r} has codebase version {version}; supported: {', '.join(SUPPORTED_VERSIONS)}")


def load_info(root: Path) -> dict:
    info = load_json(root / INFO_PATH)
    for ft in info["features"].values():
        ft["shape"] = tuple(ft["shape"])
    return info


def load_tasks(root: Path, version: str) -> tuple[dict[int, str], dict[str, int]]:
    if version == "v3.0":
        import pyarrow.parquet as pq
        t = pq.read_table(root / V30_TASKS_PATH).to_pandas()
        if "task" not in t.columns:            # the task string is the index column in v3.0 files
            t = t.reset_index().rename(columns={t.index.name or "index": "task"})
        tasks = {int(r.task_index): str(r.task) for r in t.itertuples()}
    else:
        tasks = {int(r["task_index"]): r["task"] for r in load_jsonlines(root / TASKS_PATH)}
    return tasks, {v: k for k, v in tasks.items()}


def load_episodes(root: Path, version: str) -> dict[int, dict]:
    """``episode_index -> row``; v3.0 rows also carry the file placement and video time offsets."""
    if version == "v3.0":
        import pyarrow.parquet as pq
        files = sorted((root / V30_EPISODES_DIR).glob("chunk-*/file-*.parquet"))
        out: dict[int, dict] = {}
        for f in files:
            for row in pq.read_table(f).to_pylist():
                row = {k: v for k, v in row.items() if not k.startswith("stats/")}
                out[int(row["episode_index"])] = row
        return out
    return {int(r["episode_index"]): r for r in load_jsonlines(root / EPISODES_PATH)}


def load_stats(root: Path, version: str) -> dict | None:
    """Dataset-level stats; v2.1 aggregates its per-episode records."""
    if version == "v2.1" and (root / EPISODES_STATS_PATH).exists():
        from .compute_stats import aggregate_stats
        per_ep = [cast_stats_to_numpy(r["stats"]) for r in load_jsonlines(root / EPISODES_STATS_PATH)]
        return aggregate_stats(per_ep) if per_ep else None
    if (root / STATS_PATH).exists():
        return cast_stats_to_numpy(unflatten_dict(flatten_dict(load_json(root / STATS_PATH))))
    return None


def load_episodes_stats(root: Path) -> dict[int, dict]:
    if not (root / EPISODES_STATS_PATH).exists():
        return {}
    return {int(r["episode_index"]): cast_stats_to_numpy(r["stats"]) for r in load_jsonlines(root / EPISODES_STATS_PATH)}


def get_episode_data_index(episodes: dict[int, dict], selected: list[int] | None = None) -> dict[str, torch.Tensor]:
    lengths = {i: int(e["length"]) for i, e in episodes.items()}
    if selected is not None:
        lengths = {i: lengths[i] for i in selected}
    cum = list(accumulate(lengths.values()))
    return {"from": torch.LongTensor([0] + cum[:-1]), "to": torch.LongTensor(cum)}


def dataset_to_policy_features(features: dict[str, dict]) -> dict[str, PolicyFeature]:
    """LeRobot feature dict -> policy features (images become channel-first VISUAL features)."""
    out: dict[str, PolicyFeature] = {}
    for key, ft in features.items():
        shape = tuple(ft["shape"])
        if ft["dtype"] in ("image", "video"):
            if len(shape) != 3:
                raise ValueError(f"Number of dimensions of {key} != 3 (shape={shape})")
            names = ft.get("names") or []
            if names and names[2] in ("channel", "channels"):
                shape = (shape[2], shape[0], shape[1])
            out[key] = PolicyFeature(FeatureType.VISUAL, shape)
        elif key == "observation.environment_state":
            out[key] = PolicyFeature(FeatureType.ENV, shape)
        elif key.startswith("observation"):
            out[key] = PolicyFeature(FeatureType.STATE, shape)
        elif key.startswith("action"):
            out[key] = PolicyFeature(FeatureType.ACTION, shape)
    return out


def validate_frame(frame: dict, features: dict[str, dict]) -> None:
    """A frame handed to the recorder must hold exactly the declared non-default features with matching shapes."""
    expected = set(features) - set(DEFAULT_FEATURES)
    actual = set(frame) - {"task", "timestamp"}
    msgs = []
    if expected - actual:
        msgs.append(f"missing features: {sorted(expected - actual)}")
    if actual - expected:
        msgs.append(f"extra features: {sorted(actual - expected)}")
    for k in expected & actual:
        ft, v = features[k], frame[k]
        if ft["dtype"] in ("image", "video"):
            arr = np.asarray(v)
            c_first = (arr.shape[-1], *arr.shape[:-1]) if arr.ndim == 3 else arr.shape
            if tuple(arr.shape) != tuple(ft["shape"]) and tuple(c_first) != tuple(ft["shape"]) and \
                    (arr.shape[1], arr.shape[2], arr.shape[0]) != tuple(ft["shape"]):
                msgs.append(f"feature {k!r}: image shape {arr.shape} does not match {ft['shape']}")
        elif ft["dtype"] != "string":
            arr = np.asarray(v)
            if tuple(arr.shape) != tuple(ft["shape"]):
                msgs.append(f"feature {k!r}: shape {arr.shape} != {tuple(ft['shape'])}")
    if msgs:
        raise ValueError("invalid frame: " + "; ".join(msgs))


def cycle(iterable) -> Iterator:
    """Endless iteration that restarts the iterable (fresh shuffles) instead of caching its items."""
    it = iter(iterable)
    while True:
        try:
            yield next(it)
        except StopIteration:
            it = iter(iterable)


def hf_transform_to_torch(value: Any) -> Any:
    if isinstance(value, np.ndarray):
        return torch.from_numpy(value)
    if isinstance(value, (int, float, np.integer, np.floating)):
        return torch.tensor(value)
    return value


def check_timestamps_sync(timestamps: np.ndarray, episode_indices: np.ndarray, episode_data_index: dict,
                          fps: float, tolerance_s: float, raise_value_error: bool = True) -> bool:
    """Consecutive frames of one episode must be ``1 / fps`` apart within ``tolerance_s`` (differences across an
    episode boundary are not looked at).  A recording with dropped or duplicated frames makes every "``k`` steps ahead"
    lookup land on the wrong instant, so it is refused at load time with the offending pairs
    (reference ``src/opentau/datasets/utils.py:1265-1339``)."""
    timestamps, episode_indices = np.asarray(timestamps, np.float64), np.asarray(episode_indices)
    if timestamps.shape != episode_indices.shape:
        raise ValueError(f"timestamps and episode_indices must have the same shape, got {timestamps.shape} and "
                         f"{episode_indices.shape}")
    if len(timestamps) < 2:
        return True
    diffs = np.diff(timestamps)
    ok = np.abs(diffs - 1.0 / fps) <= tolerance_s
    inside = np.ones(len(diffs), bool)
    ends = np.asarray(episode_data_index["to"], np.int64)[:-1] - 1          # last frame of every episode but the last
    inside[ends[(ends >= 0) & (ends < len(diffs))]] = False
    bad = np.flatnonzero(~ok & inside)
    if bad.size == 0:
        return True
    if raise_value_error:
        shown = [{"timestamps": [float(timestamps[i]), float(timestamps[i + 1])], "diff": float(diffs[i]),
                  "episode_index": int(episode_indices[i])} for i in bad[:10]]
        raise ValueError(f"{bad.size} pair(s) of consecutive frames are not 1/fps = {1.0 / fps:.6f} s apart within "
                         f"tolerance_s={tolerance_s}: the recording dropped or duplicated frames, or the tolerance is "
                         f"too tight for its clock.  First offenders: {shown}")
    return False


def validate_episode_buffer(episode_buffer: dict, total_episodes: int, features: dict,
                            deferred_features: set[str] | None = None) -> None:
    """An episode buffer about to be saved: it has ``size`` and ``task``, is not empty, continues the episode numbering,
    and holds exactly the dataset's features (those whose data arrives later, e.g. deferred videos, may be absent)."""
    for key in ("size", "task"):
        if key not in episode_buffer:
            raise ValueError(f"{key} key not found in episode_buffer")
    if episode_buffer["episode_index"] != total_episodes:
        raise NotImplementedError(f"episode_index {episode_buffer['episode_index']} does not continue the dataset "
                                  f"({total_episodes} episodes so far): out-of-order episodes are not supported")
    if episode_buffer["size"] == 0:
        raise ValueError("You must add one or several frames with `add_frame` before calling `save_episode`.")
    have = set(episode_buffer) - {"task", "size"}
    want = set(features) - set(deferred_features or ())
    extra, missing = have - set(features), want - have
    if extra or missing:
        raise ValueError(f"features of the episode buffer and of the dataset differ: missing {sorted(missing)}, "
                         f"unexpected {sorted(extra)}")
