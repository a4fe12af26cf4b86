"""Label every episode of a dataset mixture with subtask boundaries, using a vision-language model.

Pipeline of the reference tool (``src/opentau/scripts/annotate_subtasks.py:156-881``): sample ``--sample-fps`` frames per
second from the episode's ``camera0`` video (name resolved through the dataset's ``data_features_name_mapping``, the
built-in mapping table, then the first video feature), shrink frames whose shorter side exceeds ``--target-size`` (scale
+ centre crop, never enlarge), send frames and timestamps to the model, store the returned
``[{"time": s, "subtask": text}, ...]`` as ``subtasks/episode_XXXXXX.json``, record ``subtask_path`` in ``info.json`` and
(by default) expand the labels into the per-frame ``response`` column.  Episodes that already have a subtask file are
skipped, so an interrupted run resumes.

The model is any ``planner.ChatClient``: the hosted OpenAI client when ``--model`` names one and the package, a key and
network access exist, or a callable handed to ``run`` (tests use a scripted one).  Frames are decoded with OpenCV.

    python -m opentau_b200.scripts.annotate_subtasks --config-path mixture.json [--sample-fps 1] [--model gpt-4o]
"""

from __future__ import annotations

import argparse
import base64
import json
import logging
import re
from pathlib import Path

import numpy as np

from ..datasets.standard_data_format_mapping import DATA_FEATURES_NAME_MAPPING
from ..datasets.utils import get_version, load_episodes, load_info, write_json
from ..planner.high_level_planner import ChatClient
from .add_subtask_response import DEFAULT_CHUNK_SIZE, process_dataset

log = logging.getLogger(__name__)
SUBTASK_TEMPLATE = "subtasks/episode_{episode_index:06d}.json"

SYSTEM_PROMPT = ("You are a robot manipulation expert. You will be shown frames sampled from one robot episode, each "
                 "with its timestamp in seconds. Split the episode into the subtasks the robot performs. "
                 "Return ONLY a JSON list, no markdown fences, no prose.")
USER_TEMPLATE = ("Task: {task}\nFrame timestamps (s): {times}\n\nReturn ONLY a valid JSON list of the form "
                 '[{{"time": <start time in seconds>, "subtask": "<short imperative description>"}}, ...] '
                 "ordered by time; the first entry starts at 0.")


# ---------------------------------------------------------------------------------------------- frames
def resize_and_center_crop(img: np.ndarray, target: int) -> np.ndarray:
    """``img`` HxWx3 uint8.  Only shrinks: shorter side -> ``target``, then a centred ``target`` square."""
    import cv2
    h, w = img.shape[:2]
    if min(h, w) <= target:
        return img
    s = target / min(h, w)
    img = cv2.resize(img, (max(target, round(w * s)), max(target, round(h * s))), interpolation=cv2.INTER_AREA)
    h, w = img.shape[:2]
    y0, x0 = (h - target) // 2, (w - target) // 2
    return img[y0:y0 + target, x0:x0 + target]


def to_b64_jpeg(img: np.ndarray, quality: int = 85) -> str:
    import cv2
    ok, buf = cv2.imencode(".jpg", np.ascontiguousarray(img[:, :, ::-1]), [cv2.IMWRITE_JPEG_QUALITY, quality])
    if not ok:
        raise RuntimeError("JPEG encoding failed")
    return base64.b64encode(buf.tobytes()).decode()


def frames_at_indices(video: Path, indices: list[int], target: int) -> dict[int, np.ndarray]:
    """One sequential pass over the file; returns RGB frames for the decode-order indices that exist."""
    import cv2
    wanted, out = set(indices), {}
    cap = cv2.VideoCapture(str(video))
    try:
        i = 0
        while wanted - set(out):
            ok, bgr = cap.read()
            if not ok:
                break
            if i in wanted:
                out[i] = resize_and_center_crop(bgr[:, :, ::-1], target)
            i += 1
    finally:
        cap.release()
    return out


def sampled_frames(video: Path, fps: float, sample_fps: float, target: int) -> tuple[list[float], list[np.ndarray]]:
    import cv2
    cap = cv2.VideoCapture(str(video))
    n = int(cap.get(cv2.CAP_PROP_FRAME_COUNT))
    cap.release()
    step = max(1, round(fps / sample_fps))
    idx = list(range(0, max(n, 1), step))
    got = frames_at_indices(video, idx, target)
    keep = [i for i in idx if i in got]
    return [i / fps for i in keep], [got[i] for i in keep]


# ---------------------------------------------------------------------------------------------- parsing
def parse_json_response(text: str):
    """Tolerates markdown fences and prose around the JSON value."""
    text = re.sub(r"^```(?:json)?|```$", "", text.strip(), flags=re.MULTILINE).strip()
    try:
        return json.loads(text)
    except json.JSONDecodeError:
        m = re.search(r"(\[.*\]|\{.*\})", text, flags=re.DOTALL)
        if m is None:
            raise
        return json.loads(m.group(1))


def coerce_subtasks(parsed) -> list[dict]:
    """Keeps well-formed entries, sorted by time; anything else is dropped."""
    out = []
    for e in parsed if isinstance(parsed, list) else []:
        if isinstance(e, dict) and "time" in e and "subtask" in e:
            try:
                out.append({"time": float(e["time"]), "subtask": str(e["subtask"]).strip()})
            except (TypeError, ValueError):
                continue
    return sorted((e for e in out if e["subtask"]), key=lambda e: e["time"])


# ---------------------------------------------------------------------------------------------- datasets
def resolve_camera0_video_key(info: dict, ds_cfg: dict) -> str | None:
    feats = info.get("features", {})
    for mapping in (ds_cfg.get("data_features_name_mapping") or {}, DATA_FEATURES_NAME_MAPPING.get(ds_cfg.get("repo_id"), {})):
        key = mapping.get("camera0")
        if key is not None:
            return key if feats.get(key, {}).get("dtype") == "video" else None
    return next((k for k, f in feats.items() if f.get("dtype") == "video"), None)


def load_datasets_from_config(path: str | Path) -> list[dict]:
    """Accepts ``{"dataset_mixture": {"datasets": [...]}}`` and ``{"datasets": [...]}``."""
    cfg = json.loads(Path(path).read_text())
    cfg = cfg.get("dataset_mixture", cfg)
    if "datasets" not in cfg:
        raise ValueError(f"{path}: no 'datasets' list")
    return list(cfg["datasets"])


def video_file(root: Path, info: dict, key: str, ep: int) -> Path:
    chunk = ep // int(info.get("chunks_size", DEFAULT_CHUNK_SIZE))
    return root / info["video_path"].format(episode_chunk=chunk, video_key=key, episode_index=ep)


def annotate_episode(client: ChatClient, root: Path, info: dict, key: str, ep: int, ep_info: dict, sample_fps: float,
                     target: int) -> bool:
    out = root / SUBTASK_TEMPLATE.format(episode_index=ep)
    if out.is_file():
        return False
    video = video_file(root, info, key, ep)
    if not video.is_file():
        log.warning("episode %d: no video at %s; skipped", ep, video)
        return False
    times, frames = sampled_frames(video, float(info["fps"]), sample_fps, target)
    if not frames:
        log.warning("episode %d: no frame decoded; skipped", ep)
        return False
    tasks = ep_info.get("tasks") or ["robot manipulation task"]
    messages = [{"role": "system", "content": SYSTEM_PROMPT},
                {"role": "user", "content": USER_TEMPLATE.format(task=tasks[0], times=[round(t, 2) for t in times])}]
    try:
        subtasks = coerce_subtasks(parse_json_response(client.complete(messages, [to_b64_jpeg(f) for f in frames])))
    except Exception as e:  # noqa: BLE001 - an unusable answer must not end a long annotation run
        log.warning("episode %d: annotation failed (%s); skipped", ep, e)
        return False
    if not subtasks:
        log.warning("episode %d: the model returned no usable subtask; skipped", ep)
        return False
    out.parent.mkdir(parents=True, exist_ok=True)
    out.write_text(json.dumps(subtasks, indent=2))
    return True


def run(datasets: list[dict], client: ChatClient, sample_fps: float = 1.0, target_size: int = 448,
        max_episodes_per_dataset: int | None = None, write_response_column: bool = True) -> dict[str, int]:
    """Returns ``{root: episodes annotated in this call}``."""
    done = {}
    for ds in datasets:
        if not ds.get("root"):
            raise ValueError(f"dataset {ds.get('repo_id')!r} has no local 'root' (no hub download offline)")
        root = Path(ds["root"]).resolve()
        info = load_info(root)
        if get_version(info) != "v2.1":
            log.warning("%s: codebase_version %s, written for v2.1", root, get_version(info))
        key = resolve_camera0_video_key(info, ds)
        if key is None:
            log.warning("%s: no camera0 video feature; skipped", root)
            continue
        episodes = load_episodes(root, get_version(info))
        n = 0
        for ep in sorted(episodes)[:max_episodes_per_dataset]:
            n += annotate_episode(client, root, info, key, ep, episodes[ep], sample_fps, target_size)
        if info.get("subtask_path") != SUBTASK_TEMPLATE:
            info["subtask_path"] = SUBTASK_TEMPLATE
            write_json(info, root / "meta" / "info.json")
        if write_response_column:
            process_dataset(root)
        done[str(root)] = n
    return done


def make_client(model: str) -> ChatClient:
    if model.startswith(("gpt", "o1", "o3", "o4")):
        from ..planner.high_level_planner import OpenAIClient
        return OpenAIClient(model)
    raise ValueError(f"no client for model {model!r} in this build: pass a ChatClient to run() "
                     "(hosted Anthropic / Gemini SDKs are not part of this environment)")


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config-path", required=True)
    ap.add_argument("--model", default="gpt-4o")
    ap.add_argument("--sample-fps", type=float, default=1.0)
    ap.add_argument("--target-size", type=int, default=448)
    ap.add_argument("--max-episodes-per-dataset", type=int, default=None)
    ap.add_argument("--no-write-response-column", dest="write_response", action="store_false", default=True)
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO)
    done = run(load_datasets_from_config(a.config_path), make_client(a.model), a.sample_fps, a.target_size,
               a.max_episodes_per_dataset, a.write_response)
    for root, n in done.items():
        log.info("%s: %d episodes annotated", root, n)


if __name__ == "__main__":
    main()
