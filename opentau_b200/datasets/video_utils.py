"""Video decode / encode with backend selection (reference ``src/opentau/datasets/video_utils.py:118-865``).

Backends, best first: ``torchcodec`` (needs its compiled extension and a system FFmpeg), ``pyav`` (PyAV), ``opencv``
(always present in this image).  ``get_safe_default_codec`` probes once per process and returns the best one that
actually loads; asking explicitly for a backend that cannot load downgrades to the next with ONE warning per process
(the decode call sits in the per-sample path of the data loader).  Every backend returns the frames nearest to the
requested timestamps as float ``(N, C, H, W)`` in [0, 1] and enforces the same contract: a query farther than
``tolerance_s`` from every decoded frame raises.  A small per-process cache keeps OpenCV capture handles open across
samples of the same episode.
"""

from __future__ import annotations

import functools
import importlib.util
import logging
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


BACKENDS = ("torchcodec", "pyav", "opencv")


@functools.cache
def _probe_backend(name: str) -> BaseException | None:
    """None when ``name`` is usable here, else the exception that says why not (cached: one probe per process)."""
    try:
        if name == "torchcodec":
            if importlib.util.find_spec("torchcodec") is None:
                return ModuleNotFoundError("torchcodec is not installed")
            from torchcodec.decoders import VideoDecoder  # noqa: F401
        elif name == "pyav":
            if importlib.util.find_spec("av") is None:
                return ModuleNotFoundError("PyAV (av) is not installed")
            import av  # noqa: F401
        elif name == "opencv":
            import cv2  # noqa: F401
        else:
            return ValueError(f"unsupported video backend: {name}")
    except (ImportError, RuntimeError, ValueError) as e:     # a compiled extension that fails to load raises any of these
        return e
    return None


def get_safe_default_codec() -> str:
    """The best decode backend that loads on this host."""
    for name in BACKENDS:
        if _probe_backend(name) is None:
            return name
    raise RuntimeError("no video decode backend is available (torchcodec, PyAV and OpenCV all failed to load)")


@functools.cache
def _warn_downgrade(asked: str, got: str) -> None:
    logging.warning("video backend %r was requested but cannot load (%s); using %r instead", asked,
                    _probe_backend(asked), got)


def resolve_backend(backend: str | None) -> str:
    """``None`` -> the best available; an explicit but unloadable backend -> the next that loads (warned once); an
    unknown name raises.  ``video_reader`` is accepted as the reference's alias of the PyAV path."""
    if backend is None:
        return get_safe_default_codec()
    if backend == "video_reader":
        backend = "pyav"
    if backend not in BACKENDS:
        raise ValueError(f"Unsupported video backend: {backend}")
    if _probe_backend(backend) is None:
        return backend
    for name in BACKENDS[BACKENDS.index(backend) + 1:]:
        if _probe_backend(name) is None:
            _warn_downgrade(backend, name)
            return name
    raise RuntimeError(f"video backend {backend!r} and every fallback failed to load")


def _check_tolerance(query: torch.Tensor, loaded: torch.Tensor, tolerance_s: float, path) -> torch.Tensor:
    """Index of the closest loaded timestamp per query; raises when any is farther than the tolerance."""
    dist = torch.cdist(query[:, None].double(), loaded[:, None].double(), p=1)
    best, idx = dist.min(1)
    if not (best <= tolerance_s + 1e-9).all():
        bad = query[best > tolerance_s + 1e-9]
        raise FrameTimestampError(
            f"query timestamps {bad.tolist()} are farther than tolerance_s={tolerance_s} from every decoded frame of "
            f"{path}: the requested timestamps do not match the video's frame times, or the tolerance is too small")
    return idx


def decode_video_frames_torchcodec(path: str | Path, timestamps: list[float], tolerance_s: float) -> torch.Tensor:
    from torchcodec.decoders import VideoDecoder
    dec = VideoDecoder(str(path), device="cpu", seek_mode="approximate")
    fps = dec.metadata.average_fps
    idx = [min(max(int(round(t * fps)), 0), dec.metadata.num_frames - 1) for t in timestamps]
    batch = dec.get_frames_at(indices=idx)
    keep = _check_tolerance(torch.tensor(timestamps), batch.pts_seconds.double(), tolerance_s, path)
    return batch.data[keep].float() / 255.0


def decode_video_frames_pyav(path: str | Path, timestamps: list[float], tolerance_s: float) -> torch.Tensor:
    """Seeks to the key frame before the first query and decodes forward to the last one."""
    import av
    first, last = min(timestamps), max(timestamps)
    frames, pts = [], []
    with av.open(str(path)) as container:
        stream = container.streams.video[0]
        container.seek(int(max(first, 0.0) / stream.time_base), stream=stream, backward=True, any_frame=False)
        for frame in container.decode(stream):
            t = float(frame.pts * stream.time_base)
            frames.append(torch.from_numpy(frame.to_ndarray(format="rgb24")))
            pts.append(t)
            if t >= last:
                break
    if not frames:
        raise FrameTimestampError(f"no frame could be decoded from {path}")
    keep = _check_tolerance(torch.tensor(timestamps), torch.tensor(pts), tolerance_s, path)
    return torch.stack(frames)[keep].permute(0, 3, 1, 2).float() / 255.0


def decode_video_frames(path: str | Path, timestamps: list[float], tolerance_s: float, backend: str | None = None,
                        fps: float | None = None) -> torch.Tensor:
    """Frames nearest to ``timestamps`` (seconds) through ``backend`` (see :func:`resolve_backend`).  The backends
    pick frames by different rules (presentation-time search vs ``round(t * fps)``), so for one file they can differ
    within ``tolerance_s``; a caller that needs one specific backend checks ``get_safe_default_codec()`` first."""
    backend = resolve_backend(backend)
    if backend == "torchcodec":
        return decode_video_frames_torchcodec(path, timestamps, tolerance_s)
    if backend == "pyav":
        return decode_video_frames_pyav(path, timestamps, tolerance_s)
    return decode_video_frames_opencv(path, timestamps, tolerance_s, fps)


def decode_video_frames_opencv(path: str | Path, timestamps: list[float], tolerance_s: float,
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


def get_video_pixel_channels(pix_fmt: str) -> int:
    """1 for grey / depth formats, 4 with an alpha plane, 3 for rgb / yuv; unknown formats raise."""
    if "gray" in pix_fmt or "depth" in pix_fmt or "monochrome" in pix_fmt:
        return 1
    if "rgba" in pix_fmt or "yuva" in pix_fmt:
        return 4
    if "rgb" in pix_fmt or "yuv" in pix_fmt:
        return 3
    raise ValueError(f"unknown pixel format {pix_fmt!r}")


def get_image_pixel_channels(image) -> int:
    """Channels of a PIL image by mode (L, LA, RGB, RGBA)."""
    try:
        return {"L": 1, "LA": 2, "RGB": 3, "RGBA": 4}[image.mode]
    except KeyError:
        raise ValueError(f"unknown image mode {image.mode!r}") from None


def resample_and_trim_video(input_path: str | Path, output_path: str | Path, target_fps: int, num_frames: int,
                            overwrite: bool = False, start_time: float | None = None) -> None:
    """Re-times a recorded video to ``target_fps`` and cuts it to exactly ``num_frames`` frames starting
    ``start_time`` seconds in (attaching a pre-recorded clip to an episode whose other signals are already stored;
    reference ``video_utils.py:711-865``, which shells out to ffmpeg).  Output frame ``k`` is the source frame
    nearest to ``start_time + k / target_fps``; a source that ends early raises."""
    import cv2
    input_path, output_path = Path(input_path), Path(output_path)
    if num_frames <= 0:
        raise ValueError(f"`num_frames` must be > 0, got {num_frames}.")
    if not input_path.is_file():
        raise FileNotFoundError(f"input video not found: {input_path}")
    if output_path.exists() and not overwrite:
        return
    cap = cv2.VideoCapture(str(input_path))
    if not cap.isOpened():
        raise OSError(f"cannot open {input_path}")
    try:
        src_fps = float(cap.get(cv2.CAP_PROP_FPS)) or float(target_fps)
        n_src = int(cap.get(cv2.CAP_PROP_FRAME_COUNT))
        t0 = float(start_time or 0.0)
        want = [int(round((t0 + k / target_fps) * src_fps)) for k in range(num_frames)]
        if want[-1] > n_src:                                  # one frame of slack for container rounding
            raise ValueError(f"{input_path} has {n_src} frames at {src_fps:.2f} fps: too short for {num_frames} frames "
                             f"at {target_fps} fps from {t0:.2f}s")
        want = [min(i, n_src - 1) for i in want]
        w, h = int(cap.get(cv2.CAP_PROP_FRAME_WIDTH)), int(cap.get(cv2.CAP_PROP_FRAME_HEIGHT))
        output_path.parent.mkdir(parents=True, exist_ok=True)
        wr = cv2.VideoWriter(str(output_path), cv2.VideoWriter_fourcc(*"mp4v"), float(target_fps), (w, h))
        if not wr.isOpened():
            raise OSError(f"cannot open a video writer for {output_path}")
        try:
            cur, frame = -1, None
            for i in want:
                if i != cur:
                    if i != cur + 1:
                        cap.set(cv2.CAP_PROP_POS_FRAMES, i)
                    ok, frame = cap.read()
                    if not ok:
                        raise ValueError(f"could not decode frame {i} of {input_path}")
                    cur = i
                wr.write(frame)
        finally:
            wr.release()
    finally:
        cap.release()


def close_all() -> None:
    with _CACHE_LOCK:
        while _CAPTURES:
            _, c = _CAPTURES.popitem()
            c.release()
