"""Attach metadata to a LeRobot dataset (reference ``src/opentau/scripts/attach_metadata.py``,
``add_subtask_response.py``).

Two entry points:

* :func:`attach_annotations` / ``--annotations`` + ``--copy-to``: the strict, copy-only pipeline.  A JSON LIST with one
  object per episode, ``{"episode_id": 0, "quality": 3, "segments": [{"start": 0, "subtask": "...", "success": false},
  ...]}``, is validated in full before anything is written (it must cover the dataset's episodes exactly; ``start`` is an
  int FRAME index, the first is 0, they strictly increase and stay below the episode length; ``quality`` is an int in
  1..5; ``success`` a bool).  The copy's parquet files gain ``response`` (the current segment's subtask), ``memory`` (a
  running summary written by a chat model, or ``memory<frame>`` placeholders under ``--skip-memory``) and ``mistake``
  (1 where the segment failed); ``meta/info.json`` gains the three features, ``meta/episodes.jsonl`` gains ``quality`` and
  ``segments`` (start frames).  Statistics files are left alone: the new columns carry none.  The source is never touched.
* :func:`attach` / ``--metadata``: in-place labels keyed by episode (quality / speed / success flags, segments with
  explicit ends), described next.

Input: JSON ``{"episodes": {"<index>": {"quality": 4, "success": true, "speed": 3,
"segments": [[0, 40, "reach the cup"], [40, 95, "lift the cup"]]}}}``.  Episode-level fields go into
``meta/episodes.jsonl``; segment labels become a ``response`` string column of the episode's parquet file.

    python -m opentau_b200.scripts.attach_metadata --root /path/to/dataset --metadata labels.json
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

from ..datasets.utils import EPISODES_PATH, INFO_PATH, load_info, load_jsonlines, write_json, write_jsonlines


def attach(root: str | Path, labels: dict) -> dict:
    import pyarrow as pa
    import pyarrow.parquet as pq
    root = Path(root)
    info = load_info(root)
    if str(info.get("codebase_version", "")).lstrip("v") not in ("2.0", "2.1"):
        raise ValueError("attach_metadata edits the per-episode layout (v2.0 / v2.1)")
    eps = load_jsonlines(root / EPISODES_PATH)
    by_idx = {int(e["episode_index"]): e for e in eps}
    touched = {"episodes": 0, "frames_labelled": 0}
    for key, lab in labels.get("episodes", {}).items():
        ep = by_idx[int(key)]
        for f in ("quality", "speed", "success", "sum_reward"):
            if f in lab:
                ep[f] = lab[f]
        segs = lab.get("segments")
        if segs:
            # the metadata keeps the START frame of every segment (a segment ends where the next one starts, the
            # last one at the episode's end): the format the dataset reader's segment tables are built from
            ep["segments"] = [int(s) for s, *_ in segs]
            path = root / info["data_path"].format(episode_chunk=int(key) // info.get("chunks_size", 1000), episode_index=int(key))
            table = pq.read_table(path)
            resp = [""] * table.num_rows
            for s, e, *text in segs:
                for i in range(int(s), min(int(e), table.num_rows)):
                    resp[i] = text[0] if text else ""
            if "response" in table.column_names:
                table = table.drop(["response"])
            pq.write_table(table.append_column("response", pa.array(resp)), path)
            touched["frames_labelled"] += sum(1 for r in resp if r)
        touched["episodes"] += 1
    write_jsonlines([by_idx[k] for k in sorted(by_idx)], root / EPISODES_PATH)
    if any("segments" in lab for lab in labels.get("episodes", {}).values()):
        info["features"]["response"] = {"dtype": "string", "shape": (1,), "names": None}
        info["features"] = {k: {**v, "shape": list(v["shape"])} for k, v in info["features"].items()}
        write_json(info, root / INFO_PATH)
    return touched


RESPONSE_COL, MEMORY_COL, MISTAKE_COL = "response", "memory", "mistake"


def copy_dataset_tree(src: Path, dst: Path, *, overwrite: bool) -> None:
    import shutil
    if dst.exists():
        if not overwrite:
            raise FileExistsError(f"output path already exists: {dst}; pass --overwrite to replace it")
        shutil.rmtree(dst)
    dst.parent.mkdir(parents=True, exist_ok=True)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns(".DS_Store"))


def _is_int(x) -> bool:
    return isinstance(x, int) and not isinstance(x, bool)


def validate_segments(segments, ep_id: int, ep_length: int) -> None:
    if not isinstance(segments, list) or not segments:
        raise ValueError(f"Episode {ep_id} must have a non-empty 'segments' list.")
    prev = -1
    for k, seg in enumerate(segments):
        if not isinstance(seg, dict):
            raise ValueError(f"Episode {ep_id} segment {k} must be an object.")
        for key in ("start", "subtask", "success"):
            if key not in seg:
                raise ValueError(f"Episode {ep_id} segment {k} missing required key '{key}'.")
        start = seg["start"]
        if not _is_int(start):
            raise ValueError(f"Episode {ep_id} segment {k} start must be int (a frame index, not a time), got "
                             f"{type(start).__name__}.")
        if k == 0 and start != 0:
            raise ValueError(f"Episode {ep_id} first segment must start at 0, got {start}.")
        if start <= prev:
            raise ValueError(f"Episode {ep_id} segment starts must strictly increase; segment {k} start={start} <= "
                             f"previous start={prev}.")
        if start >= ep_length:
            raise ValueError(f"Episode {ep_id} segment {k} start={start} >= episode length {ep_length}.")
        if not isinstance(seg["subtask"], str):
            raise ValueError(f"Episode {ep_id} segment {k} subtask must be a string.")
        if not isinstance(seg["success"], bool):
            raise ValueError(f"Episode {ep_id} segment {k} success must be bool.")
        prev = start


def load_and_validate_annotations(data, episode_lengths: dict[int, int]) -> dict[int, dict]:
    """``{episode_id: {"quality", "segments"}}`` from the annotation list, or ``ValueError`` naming the first fault."""
    if not isinstance(data, list):
        raise ValueError("Top-level JSON must be a list of episode annotations.")
    out: dict[int, dict] = {}
    for i, entry in enumerate(data):
        if not isinstance(entry, dict):
            raise ValueError(f"Annotation entry #{i} must be an object, got {type(entry).__name__}.")
        for key in ("episode_id", "quality", "segments"):
            if key not in entry:
                raise ValueError(f"Annotation entry #{i} missing required key '{key}'.")
        ep = entry["episode_id"]
        if not _is_int(ep):
            raise ValueError(f"Annotation entry #{i} episode_id must be int, got {type(ep).__name__}.")
        if ep in out:
            raise ValueError(f"Duplicate episode_id {ep} in annotations.")
        out[ep] = {"quality": entry["quality"], "segments": entry["segments"]}
    missing, extra = sorted(set(episode_lengths) - set(out)), sorted(set(out) - set(episode_lengths))
    if missing:
        raise ValueError(f"Missing annotations for episodes: {missing[:20]}{'...' if len(missing) > 20 else ''}.")
    if extra:
        raise ValueError(f"Unknown episodes in JSON (not in dataset): {extra[:20]}{'...' if len(extra) > 20 else ''}.")
    for ep, payload in out.items():
        q = payload["quality"]
        if not _is_int(q):
            raise ValueError(f"Episode {ep} quality must be int, got {type(q).__name__}.")
        if q not in (1, 2, 3, 4, 5):
            raise ValueError(f"Episode {ep} quality must be in 1..5, got {q}.")
        validate_segments(payload["segments"], ep, episode_lengths[ep])
    return out


def build_per_frame_columns(segments: list[dict], ep_length: int, *, skip_memory: bool):
    """``(response, memory, mistake)`` lists of length ``ep_length``: a segment runs to the next one's start."""
    response, memory, mistake = [""] * ep_length, [""] * ep_length, [0] * ep_length
    starts = [s["start"] for s in segments]
    for seg, lo, hi in zip(segments, starts, starts[1:] + [ep_length]):
        for f in range(lo, hi):
            response[f] = seg["subtask"]
            memory[f] = f"memory{f}" if skip_memory else str(seg.get("memory", ""))
            mistake[f] = 0 if seg["success"] else 1
    return response, memory, mistake


def generate_memories(ann_by_ep: dict[int, dict], episode_tasks: dict[int, str], client, delay_s: float = 0.0) -> int:
    """One running memory per segment (in place), episode by episode, with the episode's task as the prompt."""
    from .pi_mem_data_generator import enrich_list
    calls = 0
    for ep in sorted(ann_by_ep):
        items = [{"subtask": s["subtask"], "success": s["success"], "prompt": episode_tasks.get(ep, "(not provided)")}
                 for s in ann_by_ep[ep]["segments"]]
        calls += enrich_list(items, client, delay_s=delay_s)
        for seg, item in zip(ann_by_ep[ep]["segments"], items):
            seg["memory"] = item["memory"]
    return calls


def attach_annotations(root: str | Path, annotations, copy_to: str | Path, *, overwrite: bool = False,
                       skip_memory: bool = False, client=None, delay_s: float = 0.0) -> dict:
    """The copy-only pipeline described in the module docstring.  ``client``: a chat client for the memories (needed
    unless ``skip_memory``); it is asked BEFORE any file is written, so a failing model leaves no half-made copy."""
    import pyarrow as pa
    import pyarrow.parquet as pq
    root, copy_to = Path(root), Path(copy_to)
    info = load_info(root)
    if str(info.get("codebase_version", "")).lstrip("v") not in ("2.0", "2.1"):
        raise ValueError("attach_metadata edits the per-episode layout (v2.0 / v2.1)")
    eps = load_jsonlines(root / EPISODES_PATH)
    lengths = {int(e["episode_index"]): int(e["length"]) for e in eps}
    ann = load_and_validate_annotations(annotations, lengths)
    calls = 0
    if not skip_memory:
        if client is None:
            raise ValueError("memory generation needs a chat client; pass --skip-memory to write placeholders")
        tasks = {int(e["episode_index"]): (e.get("tasks") or ["(not provided)"])[0] for e in eps}
        calls = generate_memories(ann, tasks, client, delay_s)
    copy_dataset_tree(root, copy_to, overwrite=overwrite)
    frames = 0
    for ep, payload in sorted(ann.items()):
        path = copy_to / info["data_path"].format(episode_chunk=ep // info.get("chunks_size", 1000), episode_index=ep)
        table = pq.read_table(path)
        if table.num_rows != lengths[ep]:
            raise ValueError(f"episode {ep}: {table.num_rows} rows on disk, {lengths[ep]} in the metadata")
        resp, mem, bad = build_per_frame_columns(payload["segments"], lengths[ep], skip_memory=skip_memory)
        keep = [c for c in table.column_names if c not in (RESPONSE_COL, MEMORY_COL, MISTAKE_COL)]
        table = table.select(keep).append_column(RESPONSE_COL, pa.array(resp, pa.string())) \
            .append_column(MEMORY_COL, pa.array(mem, pa.string())).append_column(MISTAKE_COL, pa.array(bad, pa.int64()))
        pq.write_table(table, path)
        frames += lengths[ep]
    for e in eps:
        ep = int(e["episode_index"])
        e["quality"] = ann[ep]["quality"]
        e["segments"] = [s["start"] for s in ann[ep]["segments"]]
    write_jsonlines(eps, copy_to / EPISODES_PATH)
    info["features"][RESPONSE_COL] = {"dtype": "string", "shape": (1,), "names": None}
    info["features"][MEMORY_COL] = {"dtype": "string", "shape": (1,), "names": None}
    info["features"][MISTAKE_COL] = {"dtype": "int64", "shape": (1,), "names": None}
    info["features"] = {k: {**v, "shape": list(v["shape"])} for k, v in info["features"].items()}
    write_json(info, copy_to / INFO_PATH)
    return {"episodes": len(ann), "frames": frames, "memory_calls": calls, "output": str(copy_to)}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0], formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--root", required=True, type=Path)
    ap.add_argument("--metadata", type=Path, help="in-place labels keyed by episode")
    ap.add_argument("--annotations", type=Path, help="per-episode annotation LIST (copy-only pipeline)")
    ap.add_argument("--copy-to", type=Path, help="destination of the annotated copy (with --annotations)")
    ap.add_argument("--overwrite", action="store_true")
    ap.add_argument("--skip-memory", action="store_true", help="write memory<frame> placeholders, call no model")
    ap.add_argument("--model", default=None, help="chat model for the memories (default: $OPENAI_MODEL or gpt-4o-mini)")
    ap.add_argument("--delay", type=float, default=0.0, help="seconds between model calls")
    a = ap.parse_args(argv)
    if (a.metadata is None) == (a.annotations is None):
        ap.error("give exactly one of --metadata and --annotations")
    if a.metadata is not None:
        print(json.dumps(attach(a.root, json.loads(a.metadata.read_text()))))
        return
    if a.copy_to is None:
        ap.error("--annotations is copy-only: --copy-to is required")
    client = None
    if not a.skip_memory:
        import os
        from ..planner.high_level_planner import OpenAIClient
        client = OpenAIClient(a.model or os.environ.get("OPENAI_MODEL", "gpt-4o-mini"))
    print(json.dumps(attach_annotations(a.root, json.loads(a.annotations.read_text(encoding="utf-8")), a.copy_to,
                                        overwrite=a.overwrite, skip_memory=a.skip_memory, client=client,
                                        delay_s=a.delay)))


if __name__ == "__main__":
    main()
