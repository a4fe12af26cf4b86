"""Codebase v1.6 -> v2.0 conversion of a dataset directory on disk (reference
``src/opentau/datasets/v2/convert_dataset_v1_to_v2.py:579-765``; the batch driver over many datasets is
``batch_convert_dataset_v1_to_v2.py``).

v1.6 layout::

    data/train-*.parquet                         every episode in a few shards
    videos/<key>_episode_<000000>.mp4            flat
    meta_data/info.json                          fps, video flag, encoding
    meta_data/stats.safetensors                  "<feature>/<stat>" tensors
    meta_data/episode_data_index.safetensors

v2.0 layout::

    data/chunk-000/episode_000000.parquet        one file per episode, 1000 episodes per chunk
    videos/chunk-000/<key>/episode_000000.mp4
    meta/info.json, episodes.jsonl, tasks.jsonl, stats.json

The reference edits a hub repository through git-lfs pointers; this converter works on two local directories (the
download and upload steps are the caller's business) and therefore moves or copies the real video files.  Tasks come
from exactly one of: one description for the whole dataset, a json file ``{episode_index: description}``, or a column
of the parquet shards (``language_instruction`` wins over a single description when it is present, as in the reference).
"""

from __future__ import annotations

import argparse
import json
import logging
import shutil
from pathlib import Path

import numpy as np

from ..utils import (DEFAULT_CHUNK_SIZE, DEFAULT_PARQUET_PATH, DEFAULT_VIDEO_PATH, EPISODES_PATH, INFO_PATH, STATS_PATH,
                     TASKS_PATH, unflatten_dict, write_json, write_jsonlines)

V16 = "v1.6"
V20 = "v2.0"
V1_VIDEO_FILE = "{video_key}_episode_{episode_index:06d}.mp4"
V1_INFO_PATH = "meta_data/info.json"
V1_STATS_PATH = "meta_data/stats.safetensors"

# Open-X exports carry the description as the repr of a TensorFlow string tensor.
_TF_PREFIX, _TF_SUFFIX = "tf.Tensor(b'", "', shape=(), dtype=string)"


def clean_task(text: str) -> str:
    text = str(text)
    if text.startswith(_TF_PREFIX):
        text = text[len(_TF_PREFIX):]
    if text.endswith(_TF_SUFFIX):
        text = text[: -len(_TF_SUFFIX)]
    return text


def convert_stats_to_json(v1_dir: Path, v2_dir: Path) -> dict:
    """``meta_data/stats.safetensors`` -> ``meta/stats.json``; the round trip is checked value by value."""
    from safetensors.numpy import load_file

    flat = load_file(str(v1_dir / V1_STATS_PATH))
    serial = {k: np.asarray(v).tolist() for k, v in flat.items()}
    nested = unflatten_dict(serial)
    write_json(nested, v2_dir / STATS_PATH)
    back = json.loads((v2_dir / STATS_PATH).read_text())
    for key, value in flat.items():
        node = back
        for part in key.split("/"):
            node = node[part]
        np.testing.assert_allclose(np.asarray(node, dtype=np.float64), np.asarray(value, dtype=np.float64), rtol=1e-6)
    return nested


def _is_video_struct(field) -> bool:
    import pyarrow as pa

    if not pa.types.is_struct(field.type):
        return False
    names = {field.type.field(i).name for i in range(field.type.num_fields)}
    return names == {"path", "timestamp"}


def _is_image_struct(field) -> bool:
    import pyarrow as pa

    if not pa.types.is_struct(field.type):
        return False
    names = {field.type.field(i).name for i in range(field.type.num_fields)}
    return names == {"bytes", "path"}


def features_from_table(table, motor_names: dict[str, list[str]] | None = None) -> dict[str, dict]:
    """v2 feature descriptions from the arrow schema of the v1 shards."""
    import pyarrow as pa

    features: dict[str, dict] = {}
    for field in table.schema:
        key, typ = field.name, field.type
        if _is_video_struct(field):
            features[key] = {"dtype": "video", "shape": None, "names": ["height", "width", "channels"]}
        elif _is_image_struct(field):
            shape = None
            first = table.column(key)[0].as_py()
            if first and first.get("bytes"):
                import io

                from PIL import Image

                with Image.open(io.BytesIO(first["bytes"])) as im:
                    shape = (im.height, im.width, len(im.getbands()))
            features[key] = {"dtype": "image", "shape": shape, "names": ["height", "width", "channels"]}
        elif pa.types.is_list(typ) or pa.types.is_fixed_size_list(typ) or pa.types.is_large_list(typ):
            length = len(table.column(key)[0].as_py())
            names = (motor_names or {}).get(key) or [f"motor_{i}" for i in range(length)]
            if len(names) != length:
                raise ValueError(f"{key}: {len(names)} motor names for a vector of {length}")
            features[key] = {"dtype": str(typ.value_type), "shape": (length,), "names": {"motors": list(names)}}
        elif pa.types.is_string(typ) or pa.types.is_large_string(typ):
            features[key] = {"dtype": "string", "shape": (1,), "names": None}
        else:
            dtype = {"double": "float64", "float": "float32"}.get(str(typ), str(typ))
            features[key] = {"dtype": dtype, "shape": (1,), "names": None}
    return features


def _task_index_column(table, tasks_by_episode: dict[int, str]):
    import pyarrow as pa

    tasks = list(dict.fromkeys(tasks_by_episode.values()))
    index = {t: i for i, t in enumerate(tasks)}
    eps = table.column("episode_index").to_numpy()
    col = np.asarray([index[tasks_by_episode[int(e)]] for e in eps], dtype=np.int64)
    return table.append_column("task_index", pa.array(col)), tasks


def _task_index_from_column(table, tasks_col: str):
    import pyarrow as pa

    texts = [clean_task(t) for t in table.column(tasks_col).to_pylist()]
    tasks = list(dict.fromkeys(texts))
    index = {t: i for i, t in enumerate(tasks)}
    eps = table.column("episode_index").to_numpy()
    by_episode: dict[int, list[str]] = {}
    for e, t in zip(eps, texts):
        seen = by_episode.setdefault(int(e), [])
        if t not in seen:
            seen.append(t)
    table = table.append_column("task_index", pa.array(np.asarray([index[t] for t in texts], dtype=np.int64)))
    return table.drop_columns([tasks_col]), tasks, by_episode


def split_parquet_by_episodes(table, total_episodes: int, out_dir: Path) -> list[int]:
    """One parquet file per episode under ``data/chunk-XXX/``; returns the episode lengths."""
    import pyarrow.compute as pc
    import pyarrow.parquet as pq

    lengths = []
    for ep in range(total_episodes):
        path = out_dir / DEFAULT_PARQUET_PATH.format(episode_chunk=ep // DEFAULT_CHUNK_SIZE, episode_index=ep)
        path.parent.mkdir(parents=True, exist_ok=True)
        part = table.filter(pc.equal(table.column("episode_index"), ep))
        lengths.append(part.num_rows)
        pq.write_table(part, path)
    return lengths


def move_videos(v1_dir: Path, v2_dir: Path, video_keys: list[str], total_episodes: int, copy: bool = True) -> int:
    """Flat ``videos/<key>_episode_<i>.mp4`` -> ``videos/chunk-XXX/<key>/episode_<i>.mp4``."""
    moved = 0
    for key in video_keys:
        for ep in range(total_episodes):
            src = v1_dir / "videos" / V1_VIDEO_FILE.format(video_key=key, episode_index=ep)
            if not src.exists():
                raise FileNotFoundError(src)
            dst = v2_dir / DEFAULT_VIDEO_PATH.format(episode_chunk=ep // DEFAULT_CHUNK_SIZE, video_key=key,
                                                     episode_index=ep)
            dst.parent.mkdir(parents=True, exist_ok=True)
            (shutil.copy2 if copy else shutil.move)(str(src), str(dst))
            moved += 1
    return moved


def convert_dataset(v1_dir: str | Path, v2_dir: str | Path, *, single_task: str | None = None,
                    tasks_path: str | Path | None = None, tasks_col: str | None = None,
                    robot_type: str = "unknown", motor_names: dict[str, list[str]] | None = None,
                    copy_videos: bool = True) -> dict:
    """Convert the v1.6 dataset in ``v1_dir`` into a v2.0 dataset in ``v2_dir``; returns the new ``info``."""
    import pyarrow as pa
    import pyarrow.parquet as pq

    v1_dir, v2_dir = Path(v1_dir), Path(v2_dir)
    if sum(x is not None for x in (single_task, tasks_path, tasks_col)) != 1:
        raise ValueError("give exactly one of single_task, tasks_path, tasks_col")
    meta_v1 = json.loads((v1_dir / V1_INFO_PATH).read_text())
    shards = sorted((v1_dir / "data").glob("*.parquet"))
    if not shards:
        raise FileNotFoundError(f"no parquet shards under {v1_dir / 'data'}")
    table = pa.concat_tables([pq.read_table(s) for s in shards])
    features = features_from_table(table, motor_names)
    video_keys = [k for k, ft in features.items() if ft["dtype"] == "video"]

    if single_task and "language_instruction" in table.column_names:
        logging.warning("'single_task' given but a 'language_instruction' column exists: using the column")
        single_task, tasks_col = None, "language_instruction"

    episode_indices = sorted({int(e) for e in table.column("episode_index").to_numpy()})
    total_episodes = len(episode_indices)
    if episode_indices != list(range(total_episodes)):
        raise ValueError("episode indices are not contiguous from 0")
    total_chunks = -(-total_episodes // DEFAULT_CHUNK_SIZE)

    if single_task:
        by_ep = dict.fromkeys(episode_indices, single_task)
        table, tasks = _task_index_column(table, by_ep)
        tasks_by_episode = {e: [t] for e, t in by_ep.items()}
    elif tasks_path:
        by_ep = {int(k): v for k, v in json.loads(Path(tasks_path).read_text()).items()}
        missing = set(episode_indices) - set(by_ep)
        if missing:
            raise ValueError(f"{tasks_path} has no task for episodes {sorted(missing)[:8]}")
        table, tasks = _task_index_column(table, by_ep)
        tasks_by_episode = {e: [by_ep[e]] for e in episode_indices}
    else:
        if tasks_col not in table.column_names:
            raise ValueError(f"column {tasks_col!r} not in the parquet shards")
        table, tasks, tasks_by_episode = _task_index_from_column(table, tasks_col)
        features.pop(tasks_col, None)
    features["task_index"] = {"dtype": "int64", "shape": (1,), "names": None}
    write_jsonlines([{"task_index": i, "task": t} for i, t in enumerate(tasks)], v2_dir / TASKS_PATH)

    if video_keys:
        if not meta_v1.get("video", False):
            raise ValueError("video-frame columns found but meta_data/info.json says video=false")
        table = table.drop_columns(video_keys)
        move_videos(v1_dir, v2_dir, video_keys, total_episodes, copy=copy_videos)
        from ..video_utils import get_video_info

        for key in video_keys:
            first = v2_dir / DEFAULT_VIDEO_PATH.format(episode_chunk=0, video_key=key, episode_index=0)
            vinfo = get_video_info(first)
            features[key]["shape"] = (vinfo.pop("video.height"), vinfo.pop("video.width"), vinfo.pop("video.channels"))
            if abs(vinfo["video.fps"] - meta_v1["fps"]) > 1e-3 * max(meta_v1["fps"], 1):
                raise ValueError(f"{key}: video fps {vinfo['video.fps']} != dataset fps {meta_v1['fps']}")
            features[key]["video_info"] = vinfo
    elif meta_v1.get("video", 0):
        raise ValueError("meta_data/info.json says video=true but no video-frame column was found")

    lengths = split_parquet_by_episodes(table, total_episodes, v2_dir)
    write_jsonlines([{"episode_index": e, "tasks": tasks_by_episode[e], "length": lengths[e]}
                     for e in episode_indices], v2_dir / EPISODES_PATH)
    info = {
        "codebase_version": V20, "robot_type": robot_type, "total_episodes": total_episodes,
        "total_frames": table.num_rows, "total_tasks": len(tasks), "total_videos": total_episodes * len(video_keys),
        "total_chunks": total_chunks, "chunks_size": DEFAULT_CHUNK_SIZE, "fps": meta_v1["fps"],
        "splits": {"train": f"0:{total_episodes}"}, "data_path": DEFAULT_PARQUET_PATH,
        "video_path": DEFAULT_VIDEO_PATH if video_keys else None,
        "features": {k: {**v, "shape": list(v["shape"]) if v["shape"] is not None else None}
                     for k, v in features.items()},
    }
    write_json(info, v2_dir / INFO_PATH)
    if (v1_dir / V1_STATS_PATH).exists():
        convert_stats_to_json(v1_dir, v2_dir)
    return info


def batch_convert(jobs: list[dict], log_path: str | Path | None = None) -> dict[str, str]:
    """Convert many datasets; one failure does not stop the others.  Each job holds the keyword arguments of
    :func:`convert_dataset` (``v1_dir``, ``v2_dir`` and one task source).  Returns ``{v1_dir: status}`` and appends
    each status line to ``log_path``."""
    import traceback

    status: dict[str, str] = {}
    for job in jobs:
        name = str(job["v1_dir"])
        try:
            convert_dataset(**job)
            status[name] = "converted"
        except Exception:  # noqa: BLE001 - the batch goes on
            status[name] = "failed\n    " + traceback.format_exc()
        if log_path:
            with open(log_path, "a") as f:
                f.write(f"{name}: {status[name]}\n")
    return status


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--v1-dir", required=True)
    ap.add_argument("--v2-dir", required=True)
    g = ap.add_mutually_exclusive_group(required=True)
    g.add_argument("--single-task")
    g.add_argument("--tasks-path")
    g.add_argument("--tasks-col")
    ap.add_argument("--robot-type", default="unknown")
    ap.add_argument("--motor-names", help="json file {feature key: [motor names]}")
    ap.add_argument("--move-videos", action="store_true", help="move instead of copy")
    a = ap.parse_args(argv)
    names = json.loads(Path(a.motor_names).read_text()) if a.motor_names else None
    info = convert_dataset(a.v1_dir, a.v2_dir, single_task=a.single_task, tasks_path=a.tasks_path,
                           tasks_col=a.tasks_col, robot_type=a.robot_type, motor_names=names,
                           copy_videos=not a.move_videos)
    print(f"converted {info['total_episodes']} episodes / {info['total_frames']} frames to {a.v2_dir}")


if __name__ == "__main__":
    main()
