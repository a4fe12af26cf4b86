"""Turn a video of a person into a LeRobot episode: frames as ``observation.images.camera``, 3-D body or hand landmarks
as ``observation.state``, and the NEXT frame's state as the action (the last frame repeats its own state).

Reference tool: ``src/opentau/scripts/human_video_to_lerobot.py:85-416`` (MediaPipe pose landmarker for third-person
``exo`` videos, 33 x 3 values; hand landmarker for first-person ``ego`` videos, 21 x 3 values per hand; optional output
rate lower than the video's).  The landmark detector is a plug-in: ``convert(..., detector=fn)`` takes any
``fn(rgb_frame) -> flat float vector``; the MediaPipe detectors are built on demand and need the ``mediapipe`` package
and its model files on disk (``--model-path``; nothing is downloaded here).

    python -m opentau_b200.scripts.human_video_to_lerobot input.mp4 ./dataset --prompt "Pick up the cup" --mode exo
"""

from __future__ import annotations

import argparse
from pathlib import Path
from typing import Callable

import numpy as np

POSE_STATE_DIM = 33 * 3
HAND_STATE_DIM_PER_HAND = 21 * 3


def landmarks_to_state(groups, dim: int, per_group: int) -> np.ndarray:
    """Flattens ``groups`` (lists of objects with ``x, y, z``) into ``dim`` floats, ``per_group`` per group; zeros
    where nothing was detected."""
    out = np.zeros(dim, np.float32)
    for gi, group in enumerate(groups or []):
        base = gi * per_group
        if base >= dim:
            break
        for j, lm in enumerate(group):
            if 3 * j + 2 >= per_group:
                break
            out[base + 3 * j: base + 3 * j + 3] = (lm.x, lm.y, lm.z)
    return out


def mediapipe_detector(mode: str, model_path: str, num_hands: int = 2) -> tuple[Callable, int]:  # pragma: no cover
    try:
        import mediapipe as mp
        from mediapipe.tasks import python as mp_tasks
        from mediapipe.tasks.python import vision
    except ImportError as e:
        raise ImportError("landmark detection needs the `mediapipe` package; pass `detector=` to convert() "
                          "to use another one") from e
    base = mp_tasks.BaseOptions(model_asset_path=model_path)
    if mode == "exo":
        det = vision.PoseLandmarker.create_from_options(vision.PoseLandmarkerOptions(base_options=base))
        return (lambda rgb: landmarks_to_state(det.detect(mp.Image(image_format=mp.ImageFormat.SRGB, data=rgb))
                                               .pose_world_landmarks[:1], POSE_STATE_DIM, POSE_STATE_DIM)), POSE_STATE_DIM
    det = vision.HandLandmarker.create_from_options(vision.HandLandmarkerOptions(base_options=base, num_hands=num_hands))
    dim = num_hands * HAND_STATE_DIM_PER_HAND
    return (lambda rgb: landmarks_to_state(det.detect(mp.Image(image_format=mp.ImageFormat.SRGB, data=rgb))
                                           .hand_world_landmarks, dim, HAND_STATE_DIM_PER_HAND)), dim


def convert(video: str | Path, output: str | Path, prompt: str, detector: Callable[[np.ndarray], np.ndarray],
            state_dim: int, fps: float | None = None, repo_id: str | None = None) -> dict:
    """One episode from one video.  ``fps`` below the video's rate keeps every ``round(video_fps / fps)``-th frame."""
    import cv2
    from ..datasets.lerobot_dataset import LeRobotDataset
    cap = cv2.VideoCapture(str(video))
    if not cap.isOpened():
        raise FileNotFoundError(f"cannot open {video}")
    vfps = float(cap.get(cv2.CAP_PROP_FPS)) or 30.0
    step = max(1, round(vfps / fps)) if fps else 1
    frames, states, i = [], [], 0
    while True:
        ok, bgr = cap.read()
        if not ok:
            break
        if i % step == 0:
            rgb = np.ascontiguousarray(bgr[:, :, ::-1])
            frames.append(rgb)
            states.append(np.asarray(detector(rgb), np.float32).reshape(state_dim))
        i += 1
    cap.release()
    if not frames:
        raise ValueError(f"no frame decoded from {video}")
    h, w = frames[0].shape[:2]
    out = Path(output)
    ds = LeRobotDataset.create(repo_id or out.name, fps=int(round(vfps / step)), root=out, robot_type="human", features={
        "observation.images.camera": {"dtype": "video", "shape": (h, w, 3), "names": ["height", "width", "channel"]},
        "observation.state": {"dtype": "float32", "shape": (state_dim,), "names": None},
        "action": {"dtype": "float32", "shape": (state_dim,), "names": None}}, use_videos=True, image_writer_threads=2)
    for t, (img, st) in enumerate(zip(frames, states)):
        ds.add_frame({"observation.images.camera": img, "observation.state": st,
                      "action": states[min(t + 1, len(states) - 1)], "task": prompt})
    ds.save_episode()
    ds.stop_image_writer()
    return {"frames": len(frames), "fps": int(round(vfps / step)), "state_dim": state_dim}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("video")
    ap.add_argument("output")
    ap.add_argument("--prompt", required=True)
    ap.add_argument("--mode", choices=["exo", "ego"], default="exo")
    ap.add_argument("--model-path", required=True, help="MediaPipe .task model file on disk")
    ap.add_argument("--num-hands", type=int, default=2)
    ap.add_argument("--fps", type=float, default=None)
    a = ap.parse_args(argv)
    det, dim = mediapipe_detector(a.mode, a.model_path, a.num_hands)
    print(convert(a.video, a.output, a.prompt, det, dim, a.fps))


if __name__ == "__main__":
    main()
