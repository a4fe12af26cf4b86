"""Flag failed subtask segments with a vision-language model: adds a per-frame ``mistake`` column.

Behaviour of the reference tool (``src/opentau/scripts/annotate_mistakes.py:128-633``): the per-frame ``response``
column (written by ``annotate_subtasks``) is cut into contiguous runs of one label; for each run the LAST frame of the
``camera0`` video and the label go to the model, which answers ``{"success": bool, "reason": str}``.  A reported failure
sets ``mistake = 1`` on every row of the run; success, an unparsable answer, a failed call or an undecodable frame leave
0.  Episodes that already carry the column are skipped (resumable); episodes without ``response`` are skipped with a
warning.  ``mistake`` is registered in ``info.json`` as an int64 feature.

    python -m opentau_b200.scripts.annotate_mistakes --config-path mixture.json [--model gpt-4o]
"""

from __future__ import annotations

import argparse
import logging
import re
from pathlib import Path

import pyarrow as pa
import pyarrow.parquet as pq

from ..datasets.utils import get_version, load_episodes, load_info
from ..planner.high_level_planner import ChatClient
from .add_subtask_response import episode_parquet, register_feature, replace_column
from .annotate_subtasks import (frames_at_indices, load_datasets_from_config, make_client, parse_json_response,
                                resolve_camera0_video_key, to_b64_jpeg, video_file)

log = logging.getLogger(__name__)

SYSTEM_PROMPT = ("You are a robot manipulation expert. You will be shown the final frame of a robot attempting a single "
                 "subtask. Decide whether the robot completed the subtask successfully at that frame. "
                 "Return ONLY a JSON object, no markdown fences, no prose.")
USER_TEMPLATE = ("Task: {task}\nSubtask: {subtask}\n\nThe image is the final frame of the robot's attempt at the subtask "
                 'above. Was the subtask completed successfully?\n\nReturn ONLY {{"success": true, "reason": "..."}} or '
                 '{{"success": false, "reason": "..."}}')


def parse_success_response(text: str) -> bool:
    """Raises on an answer without a readable verdict."""
    try:
        v = parse_json_response(text)
        if isinstance(v, dict) and isinstance(v.get("success"), bool):
            return v["success"]
    except ValueError:
        pass
    m = re.search(r'"?success"?\s*[:=]\s*(true|false)', text, flags=re.IGNORECASE)
    if m is None:
        raise ValueError(f"no success verdict in {text[:80]!r}")
    return m.group(1).lower() == "true"


def find_response_runs(responses: list) -> list[tuple[int, int, str]]:
    """``(first row, last row, label)`` of every contiguous run of one non-empty label."""
    runs, start = [], 0
    for i in range(1, len(responses) + 1):
        if i == len(responses) or responses[i] != responses[start]:
            if responses and responses[start]:
                runs.append((start, i - 1, str(responses[start])))
            start = i
    return runs


def query_success(client: ChatClient, task: str, subtask: str, frame) -> tuple[bool, bool]:
    """``(success, call_ok)``; any failure of the call or of the parse counts as success (no mistake flagged)."""
    messages = [{"role": "system", "content": SYSTEM_PROMPT},
                {"role": "user", "content": USER_TEMPLATE.format(task=task, subtask=subtask)}]
    try:
        return parse_success_response(client.complete(messages, [to_b64_jpeg(frame)])), True
    except Exception as e:  # noqa: BLE001
        log.warning("verdict for %r unavailable (%s); treated as success", subtask, e)
        return True, False


def annotate_episode(client: ChatClient, root: Path, info: dict, key: str, ep: int, ep_info: dict,
                     target: int) -> tuple[bool, int, int]:
    """``(rewritten, failed calls, undecodable frames)``."""
    path = episode_parquet(root, info, ep)
    if not path.is_file():
        return False, 0, 0
    names = pq.read_metadata(path).schema.names
    if "mistake" in names:
        return False, 0, 0
    if "response" not in names:
        log.warning("episode %d: no 'response' column (annotate subtasks first); skipped", ep)
        return False, 0, 0
    responses = pq.read_table(path, columns=["response"]).column("response").to_pylist()
    runs = find_response_runs(responses)
    if not runs:
        log.warning("episode %d: 'response' holds no label; skipped", ep)
        return False, 0, 0
    video = video_file(root, info, key, ep)
    if not video.is_file():
        log.warning("episode %d: no video at %s; skipped", ep, video)
        return False, 0, 0
    frames = frames_at_indices(video, [last for _, last, _ in runs], target)
    task = (ep_info.get("tasks") or ["robot manipulation task"])[0]
    mistakes, bad_calls, missing = [0] * len(responses), 0, 0
    for first, last, subtask in runs:
        if last not in frames:
            missing += 1
            continue
        success, ok = query_success(client, task, subtask, frames[last])
        bad_calls += not ok
        if not success:
            mistakes[first:last + 1] = [1] * (last + 1 - first)
    replace_column(path, "mistake", pa.array(mistakes, type=pa.int64()))
    return True, bad_calls, missing


def run(datasets: list[dict], client: ChatClient, target_size: int = 448,
        max_episodes_per_dataset: int | None = None) -> dict[str, int]:
    done = {}
    for ds in datasets:
        if not ds.get("root"):
            raise ValueError(f"dataset {ds.get('repo_id')!r} has no local 'root'")
        root = Path(ds["root"]).resolve()
        info = load_info(root)
        key = resolve_camera0_video_key(info, ds)
        if key is None:
            log.warning("%s: no camera0 video feature; skipped", root)
            continue
        episodes = load_episodes(root, get_version(info))
        n = 0
        for ep in sorted(episodes)[:max_episodes_per_dataset]:
            rewritten, bad, missing = annotate_episode(client, root, info, key, ep, episodes[ep], target_size)
            n += rewritten
            if bad or missing:
                log.warning("episode %d: %d failed calls, %d undecodable frames (left at mistake=0)", ep, bad, missing)
        if n:
            register_feature(root, info, "mistake", "int64")
        done[str(root)] = n
    return done


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config-path", required=True)
    ap.add_argument("--model", default="gpt-4o")
    ap.add_argument("--target-size", type=int, default=448)
    ap.add_argument("--max-episodes-per-dataset", type=int, default=None)
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO)
    for root, n in run(load_datasets_from_config(a.config_path), make_client(a.model), a.target_size,
                       a.max_episodes_per_dataset).items():
        log.info("%s: %d episodes annotated", root, n)


if __name__ == "__main__":
    main()
