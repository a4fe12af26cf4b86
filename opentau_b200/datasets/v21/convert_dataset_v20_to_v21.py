"""Codebase v2.0 -> v2.1: per-episode statistics (``meta/episodes_stats.jsonl``) replace the dataset-level
``meta/stats.json`` (reference ``src/opentau/datasets/v21/convert_dataset_v20_to_v21.py``; the per-episode work and
the check against the old statistics are in ``convert_stats.py`` beside this file; the metadata repair
``v21/_remove_language_instruction.py:33-85``; the driver over many datasets
``v21/batch_convert_dataset_v20_to_v21.py``).  Everything works on dataset directories on disk."""

from __future__ import annotations

import argparse
from pathlib import Path

from ..utils import EPISODES_PATH, INFO_PATH, STATS_PATH, load_info, load_jsonlines, write_json
from .convert_stats import check_aggregate_stats, convert_stats, write_episodes_stats


def fix_language_instruction(root: str | Path) -> str:
    """Some v2.0 exports list a ``language_instruction`` feature in ``meta/info.json`` that no parquet file holds.
    Drop it from the metadata; any other disagreement between metadata and parquet columns is an error."""
    import pyarrow.parquet as pq
    root = Path(root)
    info = load_info(root)
    first = root / info["data_path"].format(episode_chunk=0, episode_index=0)
    in_parquet = set(pq.read_schema(first).names)
    in_meta = {k for k, ft in info["features"].items() if ft["dtype"] != "video"}
    if in_parquet - in_meta:
        raise ValueError(f"in parquet but not in info.json: {sorted(in_parquet - in_meta)}")
    extra = in_meta - in_parquet
    if not extra:
        return "skipped (no difference)"
    if extra != {"language_instruction"}:
        raise ValueError(f"in info.json but not in parquet: {sorted(extra)}")
    info["features"].pop("language_instruction")
    write_json(info, root / INFO_PATH)
    return "removed 'language_instruction'"


def convert(root: str | Path, delete_old_stats: bool = False, num_workers: int = 0, check: bool = False) -> int:
    root = Path(root)
    info = load_info(root)
    if str(info["codebase_version"]).lstrip("v") != "2.0":
        raise ValueError(f"expected a v2.0 dataset, found {info['codebase_version']}")
    episodes = load_jsonlines(root / EPISODES_PATH)
    rows = convert_stats(root, info, episodes, num_workers)
    if check and (root / STATS_PATH).exists():
        import json
        check_aggregate_stats(rows, info["features"], json.loads((root / STATS_PATH).read_text()))
    write_episodes_stats(root, rows)
    info["codebase_version"] = "v2.1"
    info["features"] = {k: {**v, "shape": list(v["shape"])} for k, v in info["features"].items()}
    write_json(info, root / INFO_PATH)
    if delete_old_stats and (root / STATS_PATH).exists():
        (root / STATS_PATH).unlink()
    return len(rows)


def batch_convert(roots: list[str | Path], log_path: str | Path | None = None, **kw) -> dict[str, str]:
    """Convert many dataset directories; a failure is recorded and the batch goes on."""
    import traceback
    status: dict[str, str] = {}
    for root in roots:
        try:
            status[str(root)] = f"converted {convert(root, **kw)} episodes"
        except Exception:  # noqa: BLE001
            status[str(root)] = "failed\n    " + traceback.format_exc()
        if log_path:
            with open(log_path, "a") as f:
                f.write(f"{root}: {status[str(root)]}\n")
    return status


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--root", required=True, nargs="+")
    ap.add_argument("--delete-old-stats", action="store_true")
    ap.add_argument("--num-workers", type=int, default=0)
    ap.add_argument("--check", action="store_true", help="aggregated episode statistics must match meta/stats.json")
    ap.add_argument("--fix-language-instruction", action="store_true")
    a = ap.parse_args(argv)
    if a.fix_language_instruction:
        for r in a.root:
            print(f"{r}: {fix_language_instruction(r)}")
    kw = {"delete_old_stats": a.delete_old_stats, "num_workers": a.num_workers, "check": a.check}
    if len(a.root) == 1:
        print(f"converted {convert(a.root[0], **kw)} episodes")
    else:
        for r, st in batch_convert(a.root, **kw).items():
            print(f"{r}: {st.splitlines()[0]}")


if __name__ == "__main__":
    main()
