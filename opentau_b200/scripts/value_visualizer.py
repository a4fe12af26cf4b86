"""Value-function viewer: one self-contained HTML page per episode with the value curve and camera frames along it.

The reference viewer is an interactive Streamlit app (``src/opentau/scripts/value_visualizer_app.py:50-347``: timeline
scrubber over the frames of one episode next to the value curve).  There is no browser session or GUI toolkit in a
headless training box, so this tool renders the same content statically: an inline SVG of value (and normalised return,
when present) over time with markers at the sampled frames, and those frames embedded as JPEGs below it.  Both value-file
layouts are read: ``{"(episode, timestamp)": value}`` and ``{episode: [{"frame": i, "value": v, "return": r}, ...]}``
(what ``calculate_value`` writes).

    python -m opentau_b200.scripts.value_visualizer --values values.json --output viz/ [--dataset-root ds --episode 0]
"""

from __future__ import annotations

import argparse
import base64
import html
import json
from pathlib import Path

import numpy as np


def load_values(path: str | Path, fps: float | None = None) -> dict[int, list[dict]]:
    """-> ``{episode: [{"t": seconds or frame index, "value": v, "return": r | None}, ...]}`` sorted by ``t``."""
    raw = json.loads(Path(path).read_text())
    out: dict[int, list[dict]] = {}
    for k, v in raw.items():
        if isinstance(v, list):
            out[int(k)] = [{"t": e["frame"] / fps if fps else e["frame"], "value": float(e["value"]),
                            "return": e.get("return")} for e in v]
            continue
        key = str(k).strip().strip("()").replace(" ", "").split(",", 1)
        if len(key) == 2:
            out.setdefault(int(key[0]), []).append({"t": round(float(key[1]), 6), "value": float(v), "return": None})
    return {ep: sorted(rows, key=lambda r: r["t"]) for ep, rows in out.items()}


def svg_curve(rows: list[dict], marks: list[float], width: int = 900, height: int = 260) -> str:
    t = np.array([r["t"] for r in rows], float)
    series = {"value": np.array([r["value"] for r in rows], float)}
    if all(r["return"] is not None for r in rows):
        series["return"] = np.array([r["return"] for r in rows], float)
    lo = min(s.min() for s in series.values())
    hi = max(s.max() for s in series.values())
    hi = hi if hi > lo else lo + 1.0
    t1 = t[-1] if t[-1] > t[0] else t[0] + 1.0
    px = lambda x: 40 + (x - t[0]) / (t1 - t[0]) * (width - 60)            # noqa: E731
    py = lambda y: height - 30 - (y - lo) / (hi - lo) * (height - 50)       # noqa: E731
    parts = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-size="11">',
             f'<rect width="{width}" height="{height}" fill="#fff" stroke="#ccc"/>',
             f'<text x="4" y="{py(hi) + 4:.0f}">{hi:.3g}</text><text x="4" y="{py(lo) + 4:.0f}">{lo:.3g}</text>',
             f'<text x="{px(t[0]):.0f}" y="{height - 8}">{t[0]:.3g}</text>'
             f'<text x="{px(t1) - 30:.0f}" y="{height - 8}">{t1:.3g}</text>']
    for (name, ys), colour in zip(series.items(), ("#1f77b4", "#ff7f0e")):
        pts = " ".join(f"{px(a):.1f},{py(b):.1f}" for a, b in zip(t, ys))
        parts.append(f'<polyline fill="none" stroke="{colour}" stroke-width="1.5" points="{pts}"/>')
        parts.append(f'<text x="{width - 70}" y="{16 + 14 * list(series).index(name)}" fill="{colour}">{name}</text>')
    for m in marks:
        parts.append(f'<line x1="{px(m):.1f}" x2="{px(m):.1f}" y1="10" y2="{height - 30}" stroke="#999" '
                     'stroke-dasharray="3,3"/>')
    return "".join(parts) + "</svg>"


def jpeg_b64(img: np.ndarray, max_side: int = 224) -> str:
    import cv2
    h, w = img.shape[:2]
    s = max_side / max(h, w)
    if s < 1:
        img = cv2.resize(img, (round(w * s), round(h * s)), interpolation=cv2.INTER_AREA)
    ok, buf = cv2.imencode(".jpg", np.ascontiguousarray(img[:, :, ::-1]))
    return base64.b64encode(buf.tobytes()).decode() if ok else ""


def episode_frames(dataset_root: str | Path, episode: int, n: int,
                   indices: list[int] | None = None) -> list[tuple[float, np.ndarray]]:
    """``n`` evenly spaced frames (or the frames at ``indices``) ``(seconds, HxWx3 uint8)`` of the first camera of
    ``episode``, read straight from the episode's video file or, for image datasets, from the frames embedded in its
    parquet."""
    import io

    import pyarrow.parquet as pq
    from PIL import Image
    from ..datasets.utils import get_version, load_episodes, load_info
    from .add_subtask_response import episode_parquet
    from .annotate_subtasks import frames_at_indices, video_file
    root = Path(dataset_root)
    info = load_info(root)
    length = int(load_episodes(root, get_version(info))[episode]["length"])
    if indices is None:
        idx = sorted(set(np.linspace(0, length - 1, min(n, length)).round().astype(int).tolist()))
    else:
        idx = sorted({min(max(int(i), 0), length - 1) for i in indices})
    cams = [k for k, f in info["features"].items() if f["dtype"] in ("video", "image")]
    if not cams:
        return []
    key, fps = cams[0], float(info["fps"])
    if info["features"][key]["dtype"] == "video":
        got = frames_at_indices(video_file(root, info, key, episode), idx, 10**9)
        return [(i / fps, np.asarray(got[i])) for i in idx if i in got]
    col = pq.read_table(episode_parquet(root, info, episode), columns=[key]).column(key).to_pylist()
    out = []
    for i in idx:
        cell = col[i]
        data = cell.get("bytes") if isinstance(cell, dict) else None
        img = Image.open(io.BytesIO(data)) if data else Image.open(root / cell["path"])
        out.append((i / fps, np.asarray(img.convert("RGB"))))
    return out


def render(values: dict[int, list[dict]], output: str | Path, dataset_root: str | Path | None = None,
           episodes: list[int] | None = None, n_frames: int = 8) -> list[Path]:
    out = Path(output)
    out.mkdir(parents=True, exist_ok=True)
    pages = []
    for ep in episodes or sorted(values):
        rows = values[ep]
        frames = episode_frames(dataset_root, ep, n_frames) if dataset_root is not None else []
        body = [f"<h2>episode {ep}: {len(rows)} values</h2>", svg_curve(rows, [t for t, _ in frames]), "<div>"]
        for t, img in frames:
            near = min(rows, key=lambda r: abs(r["t"] - t))
            body.append(f'<figure style="display:inline-block;margin:4px"><img src="data:image/jpeg;base64,'
                        f'{jpeg_b64(img)}"/><figcaption>t={t:.2f}s value={near["value"]:.3f}</figcaption></figure>')
        body.append("</div>")
        page = out / f"episode_{ep:06d}.html"
        page.write_text(f"<html><head><meta charset='utf-8'><title>{html.escape(str(ep))}</title></head><body>"
                        + "".join(body) + "</body></html>")
        pages.append(page)
    return pages


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--values", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--dataset-root", default=None)
    ap.add_argument("--episode", type=int, nargs="*", default=None)
    ap.add_argument("--frames", type=int, default=8)
    ap.add_argument("--fps", type=float, default=None, help="turns frame indices of a calculate_value file into seconds")
    a = ap.parse_args(argv)
    for p in render(load_values(a.values, a.fps), a.output, a.dataset_root, a.episode, a.frames):
        print(p)


if __name__ == "__main__":
    main()
