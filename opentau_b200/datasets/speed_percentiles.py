"""Episode speed labels from episode LENGTH, per task (reference ``src/opentau/datasets/speed_percentiles.py:40-409``).

Within one (dataset, task) the episodes are ranked by their length in frames and each episode's length is bucketed
into one of ``{0, 10, ..., 100}`` by where it falls among the task's percentile boundaries ``p5, p15, ..., p95``:
short episodes get low labels ("fast"), long ones high labels.  The boundaries are persisted once per dataset in
``meta/speed_percentiles.jsonl``; the file's existence is the only gate.  A task with fewer than
:data:`MIN_EPISODES_FOR_PERCENTILES` DISTINCT lengths (few episodes, or all of one length) is stored with
``"percentiles": null`` and all its episodes get the neutral :data:`SPARSE_TASK_BUCKET`.

File rows: ``{"task_index": 0, "task": "pick up the red block", "n_episodes": 47, "percentiles": [120.0, ..., 340.0]}``.
"""

from __future__ import annotations

import contextlib
import logging
import os
import uuid
from collections import defaultdict
from pathlib import Path

import numpy as np

from .utils import load_jsonlines, write_jsonlines

SPEED_PERCENTILES: tuple[int, ...] = (5, 15, 25, 35, 45, 55, 65, 75, 85, 95)
#: label i = "between p_{i-1} and p_i"; 0 = below p5, 100 = at or above p95
SPEED_BUCKET_LABELS: tuple[int, ...] = (0, 10, 20, 30, 40, 50, 60, 70, 80, 90, 100)
SPEED_PERCENTILES_PATH = "meta/speed_percentiles.jsonl"
MIN_EPISODES_FOR_PERCENTILES = 10
SPARSE_TASK_BUCKET = 50          # median-equivalent: a neutral signal instead of a misleading "fast" / "slow"

_READONLY_WARNED: set[str] = set()           # one warning per read-only dataset root
_UNKNOWN_TASK_INDEX_WARNED: set[int] = set()  # one warning per task index that tasks.jsonl does not define


def compute_task_percentiles(episode_lengths_per_task: dict[int, list[int]]) -> dict[int, list[float] | None]:
    """``{task_index: [p5, ..., p95]}`` or ``None`` where the task has too few distinct lengths to rank."""
    out: dict[int, list[float] | None] = {}
    for task, lengths in episode_lengths_per_task.items():
        if len(set(lengths)) < MIN_EPISODES_FOR_PERCENTILES:
            out[task] = None
        else:
            out[task] = [float(p) for p in np.percentile(lengths, SPEED_PERCENTILES)]
    return out


def bucket_episode_length(length: int, percentiles: list[float] | None) -> int:
    """A length equal to a boundary lands in the UPPER bucket (intervals ``[p_{i-1}, p_i)``)."""
    if percentiles is None:
        return SPARSE_TASK_BUCKET
    return SPEED_BUCKET_LABELS[int(np.searchsorted(percentiles, length, side="right"))]


def episode_to_task_index(first_row_task_index: dict[int, int], valid_task_indices: set[int]) -> dict[int, int]:
    """``{episode: task_index}`` from the integer ``task_index`` of each episode's FIRST parquet row (constant inside an
    episode by construction).  Reading the integer avoids any drift between the task string in ``episodes.jsonl`` and a
    paraphrased ``tasks.jsonl``.  An index that ``tasks.jsonl`` does not define is metadata corruption: the episode is
    left out (it still trains; its speed falls back to the sparse bucket) with one warning per distinct index."""
    out: dict[int, int] = {}
    for ep, t in first_row_task_index.items():
        t = int(t)
        if t not in valid_task_indices:
            if t not in _UNKNOWN_TASK_INDEX_WARNED:
                _UNKNOWN_TASK_INDEX_WARNED.add(t)
                logging.warning("episode parquet rows reference task_index=%d which is not defined in tasks.jsonl; "
                                "episode(s) using it fall back to the sparse speed bucket (corrupt dataset metadata)", t)
            continue
        out[ep] = t
    return out


def _atomic_write_jsonlines(rows: list[dict], path: Path) -> None:
    """Temporary file with a per-writer suffix, then ``os.replace``: a reader sees the old file or the new one, never
    half of one, also when two independent jobs share the dataset root."""
    tmp = path.with_suffix(f"{path.suffix}.{uuid.uuid4().hex}.tmp")
    try:
        write_jsonlines(rows, tmp)
        os.replace(tmp, path)
    finally:
        if tmp.exists():
            with contextlib.suppress(OSError):
                tmp.unlink()


def load_or_compute_speed_percentiles(root: str | Path, episode_lengths: dict[int, int],
                                      episode_to_task: dict[int, int],
                                      task_to_task_index: dict[str, int]) -> dict[int, list[float] | None]:
    """Per-task boundaries for the dataset at ``root``.

    An existing file is trusted as it is (delete it to force a recompute); a warning is logged only when it was
    computed from FEWER episodes than this load uses (episodes were appended since).  Rows for tasks the file lacks are
    computed from this load and appended, existing rows are kept verbatim (a subset load must not overwrite boundaries
    that came from the full dataset).  Every rank computes the same values in memory; only the main process writes,
    and all ranks meet at a barrier on every path so that nobody runs ahead of a file that is being renamed.  On a
    read-only root the in-memory values are used and one warning per root is logged."""
    from ..parallel import control
    path = Path(root) / SPEED_PERCENTILES_PATH
    main = control.is_main_process()
    try:
        existing: list[dict] = []
        if path.is_file():
            existing = load_jsonlines(path)
            missing = set(episode_to_task.values()) - {int(r["task_index"]) for r in existing}
            if not missing:
                on_disk, now = sum(int(r.get("n_episodes", 0)) for r in existing), len(episode_to_task)
                if main and on_disk < now:
                    logging.warning("stale %s: on-disk percentiles were computed from %d episodes, this load has %d; "
                                    "using them as they are, delete the file to force a recompute", path, on_disk, now)
                return {int(r["task_index"]): r["percentiles"] for r in existing}
            if main:
                logging.warning("adding %d missing task(s) %s to %s; existing rows are kept", len(missing),
                                sorted(missing), path)
            todo = missing
        else:
            todo = set(episode_to_task.values())
        by_task: dict[int, list[int]] = defaultdict(list)
        for ep, t in episode_to_task.items():
            if t in todo:
                by_task[t].append(episode_lengths[ep])
        names = {i: t for t, i in task_to_task_index.items()}
        fresh = compute_task_percentiles(dict(by_task))
        rows = existing + [{"task_index": t, "task": names.get(t, ""), "n_episodes": len(by_task.get(t, [])),
                            "percentiles": fresh[t]} for t in sorted(fresh)]
        if main:
            try:
                path.parent.mkdir(parents=True, exist_ok=True)
                _atomic_write_jsonlines(rows, path)
            except OSError as exc:
                if str(root) not in _READONLY_WARNED:
                    _READONLY_WARNED.add(str(root))
                    logging.warning("could not write speed percentiles to %s (%s); using in-memory values for this run",
                                    path, exc)
        merged = {int(r["task_index"]): r["percentiles"] for r in existing}
        merged.update(fresh)
        return merged
    finally:
        control.wait_for_everyone()


def speed_bucket_by_episode(episodes: list[int], episode_lengths: dict[int, int], episode_to_task: dict[int, int],
                            percentiles_by_task: dict[int, list[float] | None]) -> dict[int, int]:
    """The lookup ``__getitem__`` uses: one label per selected episode; an unresolved task or a task missing from a
    hand-edited file gives the sparse bucket."""
    out: dict[int, int] = {}
    for ep in episodes:
        t = episode_to_task.get(ep)
        out[ep] = SPARSE_TASK_BUCKET if t is None else bucket_episode_length(episode_lengths[ep],
                                                                             percentiles_by_task.get(t))
    return out
