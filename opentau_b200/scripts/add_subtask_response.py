"""Expand per-episode subtask annotations into a per-frame ``response`` column.

Behaviour of the reference tool (``src/opentau/scripts/add_subtask_response.py:54-218``): ``meta/info.json`` names the
per-episode subtask files through a ``subtask_path`` template; every file is a list of ``{"time": seconds, "subtask":
text}``.  Subtask *i* labels the frames from ``round(time_i * fps)`` up to the start of subtask *i+1* (the last one
runs to the end of the episode, frames before the first start stay empty, starts beyond the episode are dropped with a
warning).  A missing file fills the column with empty strings.  The parquet is rewritten atomically and a ``response``
string feature is registered in ``info.json``.

    python -m opentau_b200.scripts.add_subtask_response --config_path mixture.json
"""

from __future__ import annotations

import json
import logging
import os
from pathlib import Path

import pyarrow as pa
import pyarrow.parquet as pq

from ..configs import parser
from ..configs.default import DatasetMixtureConfig
from ..datasets.utils import get_version, load_episodes, load_info, write_json

DEFAULT_CHUNK_SIZE = 1000
log = logging.getLogger(__name__)


def episode_parquet(root: Path, info: dict, ep_index: int) -> Path:
    chunk = ep_index // int(info.get("chunks_size", DEFAULT_CHUNK_SIZE))
    return root / info["data_path"].format(episode_chunk=chunk, episode_index=ep_index)


def build_response_array(subtasks: list[dict], fps: float, length: int, ep_index: int = 0) -> list[str]:
    out = [""] * length
    ordered = sorted(subtasks, key=lambda s: s["time"])
    for i, entry in enumerate(ordered):
        start = round(entry["time"] * fps)
        if start >= length:
            log.warning("episode %d: subtask %r starts at frame %d, beyond the %d frames; dropped", ep_index,
                        entry["subtask"], start, length)
            continue
        end = min(round(ordered[i + 1]["time"] * fps), length) if i + 1 < len(ordered) else length
        if end > start:
            out[start:end] = [str(entry["subtask"])] * (end - start)
    return out


def replace_column(path: Path, name: str, values: pa.Array) -> None:
    """Set / append one column and swap the file in atomically."""
    table = pq.read_table(path)
    if name in table.column_names:
        table = table.set_column(table.schema.get_field_index(name), name, values)
    else:
        table = table.append_column(name, values)
    tmp = path.with_suffix(path.suffix + ".tmp")
    try:
        pq.write_table(table, tmp)
        os.replace(tmp, path)
    finally:
        if tmp.exists():
            tmp.unlink()


def register_feature(root: Path, info: dict, name: str, dtype: str) -> None:
    if name not in info.setdefault("features", {}):
        info["features"][name] = {"dtype": dtype, "shape": [1], "names": None}
        write_json(info, root / "meta" / "info.json")


def process_dataset(root: str | Path) -> int:
    """Returns the number of episode files rewritten."""
    root = Path(root).resolve()
    if not root.is_dir():
        raise ValueError(f"dataset root does not exist: {root}")
    info = load_info(root)
    template = info.get("subtask_path")
    if template is None:
        raise ValueError(f"{root}/meta/info.json has no 'subtask_path': cannot locate the per-episode subtask files")
    episodes = load_episodes(root, get_version(info))
    done = 0
    for ep_index in sorted(episodes):
        length = int(episodes[ep_index]["length"])
        pq_path = episode_parquet(root, info, ep_index)
        if not pq_path.is_file():
            log.warning("episode %d: no parquet at %s; skipped", ep_index, pq_path)
            continue
        sub_file = root / template.format(episode_index=ep_index)
        if sub_file.is_file():
            responses = build_response_array(json.loads(sub_file.read_text()), info["fps"], length, ep_index)
        else:
            log.warning("episode %d: no subtask file at %s; response left empty", ep_index, sub_file)
            responses = [""] * length
        rows = pq.read_metadata(pq_path).num_rows
        if rows != length:
            log.warning("episode %d: parquet has %d rows, metadata says %d; using the parquet", ep_index, rows, length)
            responses = (responses + [""] * rows)[:rows]
        replace_column(pq_path, "response", pa.array(responses, type=pa.string()))
        done += 1
    register_feature(root, info, "response", "string")
    return done


@parser.wrap()
def add_subtask_response(cfg: DatasetMixtureConfig) -> None:
    from ..utils.logging_utils import init_logging
    init_logging()
    if not cfg.datasets:
        raise ValueError("no datasets in the config")
    for ds in cfg.datasets:
        if ds.root is None:
            raise ValueError(f"dataset {ds.repo_id!r} has no local 'root'")
        process_dataset(ds.root)


def main() -> None:
    add_subtask_response()


if __name__ == "__main__":
    main()
