"""Small IO helpers (reference ``src/opentau/utils/io_utils.py:30-205``)."""

from __future__ import annotations

import contextlib
import json
import warnings
from pathlib import Path
from typing import Any, TypeVar

T = TypeVar("T")


def write_video(video_path: str | Path, stacked_frames, fps: int) -> None:
    """``stacked_frames``: iterable of ``(H,W,3)`` uint8 RGB arrays -> mp4 (OpenCV)."""
    import cv2
    import numpy as np
    frames = [np.asarray(f) for f in stacked_frames]
    if not frames:
        raise ValueError("no frames to write")
    h, w = frames[0].shape[:2]
    Path(video_path).parent.mkdir(parents=True, exist_ok=True)
    wr = cv2.VideoWriter(str(video_path), cv2.VideoWriter_fourcc(*"mp4v"), float(fps), (w, h))
    for f in frames:
        wr.write(np.ascontiguousarray(f[:, :, ::-1]))
    wr.release()


def deserialize_json_into_object(fpath: Path, obj: T) -> T:
    """Loads JSON and checks that it has the same nesting / types as ``obj`` before returning it in that shape."""
    with open(fpath) as f:
        data = json.load(f)

    def walk(t: Any, d: Any) -> Any:
        if isinstance(t, dict):
            if not isinstance(d, dict) or set(t) != set(d):
                raise TypeError(f"structure mismatch: expected keys {sorted(t)}, got {sorted(d) if isinstance(d, dict) else type(d)}")
            return {k: walk(t[k], d[k]) for k in t}
        if isinstance(t, (list, tuple)):
            if not isinstance(d, list) or len(d) != len(t):
                raise TypeError("sequence length mismatch")
            out = [walk(a, b) for a, b in zip(t, d)]
            return tuple(out) if isinstance(t, tuple) else out
        if isinstance(t, float) and isinstance(d, int):
            return float(d)
        if type(t) is not type(d):
            raise TypeError(f"type mismatch: expected {type(t).__name__}, got {type(d).__name__}")
        return d

    return walk(obj, data)


def warn_once(msg: str, _seen: set = set()) -> None:  # noqa: B006
    if msg not in _seen:
        _seen.add(msg)
        warnings.warn(msg, stacklevel=2)


@contextlib.contextmanager
def silence_output_unless_error(label: str = ""):
    """Mutes this process's stdout and stderr for the block and replays what was written only if the block raises.

    The redirection is on the FILE DESCRIPTORS 1 and 2 (``os.dup2``), not on ``sys.stdout`` / ``sys.stderr``: that also
    catches what C extensions print and what logging handlers write that took a reference to the original stream at
    import time.  Meant for the banner that every simulator worker prints on import and construction (environments x
    ranks copies per evaluation).  On failure the captured bytes go to the real stderr first, prefixed with ``label``
    (e.g. ``"task=CloseFridge idx=3"``), then the exception travels on unchanged
    (reference ``src/opentau/utils/io_utils.py:41-110``)."""
    import os
    import sys
    import tempfile
    sys.stdout.flush()
    sys.stderr.flush()
    saved_out, saved_err = os.dup(1), os.dup(2)
    failed = False
    try:
        with tempfile.TemporaryFile(mode="w+b") as buf:
            try:
                os.dup2(buf.fileno(), 1)
                os.dup2(buf.fileno(), 2)
                yield
            except BaseException:
                failed = True
                raise
            finally:
                sys.stdout.flush()
                sys.stderr.flush()
                os.dup2(saved_out, 1)
                os.dup2(saved_err, 2)
                if failed:
                    buf.seek(0)
                    data = buf.read()
                    if data:
                        head = f"--- captured output ({label}) ---\n" if label else "--- captured output ---\n"
                        os.write(2, head.encode() + data + (b"" if data.endswith(b"\n") else b"\n"))
    finally:
        os.close(saved_out)
        os.close(saved_err)
