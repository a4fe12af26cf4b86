"""Attach episode-level metadata to a LeRobot dataset in place (reference ``src/opentau/scripts/attach_metadata.py``,
``add_subtask_response.py``): quality / speed labels, success flags, subtask segments, and per-frame ``response``
strings derived from the segments.

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


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--root", required=True)
    ap.add_argument("--metadata", required=True)
    a = ap.parse_args(argv)
    print(json.dumps(attach(a.root, json.loads(Path(a.metadata).read_text()))))


if __name__ == "__main__":
    main()
