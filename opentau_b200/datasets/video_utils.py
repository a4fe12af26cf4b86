"""Video decode / encode on OpenCV (reference ``src/opentau/datasets/video_utils.py:40-865`` uses torchcodec / pyav).

``decode_video_frames`` returns the frames nearest to the requested timestamps as float ``(N, C, H, W)`` in [0,1]
and enforces the same tolerance contract as the reference: a query farther than ``tolerance_s`` from every decoded
frame raises.  A small per-process cache keeps capture handles open across samples of the same episode.
"""

from __future__ import annotations

import threading
from collections import OrderedDict
from pathlib import Path

import numpy as np
import torch

_CACHE_LOCK = threading.Lock()
_CAPTURES: "OrderedDict[str, object]" = OrderedDict()
_MAX_OPEN = 16


class FrameTimestampError(ValueError):
    pass


def _capture(path: str):
    import cv2
    with _CACHE_LOCK:
        cap = _CAPTURES.pop(path, None)
        if cap is None:
            cap = cv2.VideoCapture(path)
            if not cap.isOpened():
                raise FileNotFoundError(f"cannot open video {path}")
        _CAPTURES[path] = cap
        while len(_CAPTURES) > _MAX_OPEN:
            _, old = _CAPTURES.popitem(last=False)
            old.release()
        return cap


def get_video_info(path: str | Path) -> dict:
    import cv2
    cap = _capture(str(path))
    return {"video.fps": float(cap.get(cv2.CAP_PROP_FPS)), "video.height": int(cap.get(cv2.CAP_PROP_FRAME_HEIGHT)),
            "video.width": int(cap.get(cv2.CAP_PROP_FRAME_WIDTH)), "video.channels": 3,
            "video.num_frames": int(cap.get(cv2.CAP_PROP_FRAME_COUNT)), "video.codec": "mp4v",
            "video.pix_fmt": "yuv420p", "video.is_depth_map": False, "has_audio": False}


def decode_video_frames(path: str | Path, timestamps: list[float], tolerance_s: float, backend: str | None = None,
                        fps: float | None = None) -> torch.Tensor:
    import cv2
    cap = _capture(str(path))
    vfps = fps or float(cap.get(cv2.CAP_PROP_FPS)) or 30.0
    n = int(cap.get(cv2.CAP_PROP_FRAME_COUNT))
    frames = []
    with _CACHE_LOCK:
        for ts in timestamps:
            idx = int(round(ts * vfps))
            idx = min(max(idx, 0), max(n - 1, 0))
            if abs(idx / vfps - ts) > tolerance_s + 1e-9 and not (ts < 0 or idx == n - 1):
                raise FrameTimestampError(
                    f"query timestamp {ts:.4f}s is {abs(idx / vfps - ts):.4f}s away from the nearest frame "
                    f"(tolerance {tolerance_s}) in {path}")
            if int(cap.get(cv2.CAP_PROP_POS_FRAMES)) != idx:
                cap.set(cv2.CAP_PROP_POS_FRAMES, idx)
            ok, bgr = cap.read()
            if not ok:
                raise FrameTimestampError(f"could not decode frame {idx} of {path}")
            frames.append(torch.from_numpy(np.ascontiguousarray(bgr[:, :, ::-1])))
    out = torch.stack(frames).permute(0, 3, 1, 2).float() / 255.0
    return out


def encode_video_frames(imgs_dir: str | Path, video_path: str | Path, fps: int, overwrite: bool = False) -> None:
    """PNG frames ``frame_000000.png ...`` -> mp4."""
    import cv2
    video_path = Path(video_path)
    if video_path.exists() and not overwrite:
        return
    files = sorted(Path(imgs_dir).glob("frame_*.png"))
    if not files:
        raise FileNotFoundError(f"no frames under {imgs_dir}")
    video_path.parent.mkdir(parents=True, exist_ok=True)
    first = cv2.imread(str(files[0]))
    h, w = first.shape[:2]
    wr = cv2.VideoWriter(str(video_path), cv2.VideoWriter_fourcc(*"mp4v"), float(fps), (w, h))
    if not wr.isOpened():
        raise RuntimeError(f"cannot open a video writer for {video_path}")
    for f in files:
        wr.write(cv2.imread(str(f)))
    wr.release()


def close_all() -> None:
    with _CACHE_LOCK:
        while _CAPTURES:
            _, c = _CAPTURES.popitem()
            c.release()
