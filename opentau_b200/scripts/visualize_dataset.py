"""``opentau-dataset-viz``: inspect an episode of a LeRobot dataset without a display
(reference ``src/opentau/scripts/visualize_dataset.py`` streams to a rerun viewer).

Writes, for one episode, a contact sheet of evenly spaced frames per camera (PNG), the state and action
trajectories as line plots rendered with OpenCV (PNG) and a JSON summary (task, length, per-dimension ranges).

    opentau-dataset-viz --repo-id user/data --root /path/to/data --episode 3 --output viz_out
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import numpy as np


def plot_lines(series: np.ndarray, title: str, width: int = 960, height: int = 360) -> np.ndarray:
    """``series (T, D)`` -> RGB image with one polyline per dimension."""
    import cv2
    img = np.full((height, width, 3), 255, np.uint8)
    T, D = series.shape
    lo, hi = float(series.min()), float(series.max())
    span = hi - lo if hi > lo else 1.0
    xs = np.linspace(40, width - 10, T)
    for d in range(D):
        col = tuple(int(c) for c in np.array([(37 * d) % 200, (91 * d + 60) % 200, (151 * d + 120) % 200]))
        ys = height - 30 - (series[:, d] - lo) / span * (height - 60)
        pts = np.stack([xs, ys], 1).astype(np.int32).reshape(-1, 1, 2)
        cv2.polylines(img, [pts], False, col, 1, cv2.LINE_AA)
    cv2.putText(img, f"{title}  [{lo:.3g}, {hi:.3g}]", (40, 20), cv2.FONT_HERSHEY_SIMPLEX, 0.5, (0, 0, 0), 1, cv2.LINE_AA)
    return img


def contact_sheet(frames: list[np.ndarray], cols: int = 4) -> np.ndarray:
    h, w = frames[0].shape[:2]
    rows = -(-len(frames) // cols)
    sheet = np.zeros((rows * h, cols * w, 3), np.uint8)
    for i, f in enumerate(frames):
        r, c = divmod(i, cols)
        sheet[r * h:(r + 1) * h, c * w:(c + 1) * w] = f
    return sheet


def visualize_episode(dataset, episode: int, out_dir: str | Path, n_frames: int = 8) -> dict:
    import cv2
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    i = dataset.epi2idx[episode]
    s, e = int(dataset.episode_data_index["from"][i]), int(dataset.episode_data_index["to"][i])
    picks = np.unique(np.linspace(s, e - 1, n_frames).astype(int))
    summary = {"episode": episode, "length": e - s, "task": dataset._resolve_task(int(dataset._numeric["task_index"][s])), "files": []}
    was = dataset.standardize
    dataset.standardize = False
    try:
        for cam in dataset.meta.camera_keys:
            frames = []
            for idx in picks:
                item = dataset[int(idx)]
                img = item[cam]
                img = img[-1] if img.dim() == 4 else img
                frames.append((img.permute(1, 2, 0).float().clamp(0, 1).numpy() * 255).astype(np.uint8))
            f = out / f"episode_{episode:06d}_{cam.replace('.', '_')}.png"
            cv2.imwrite(str(f), contact_sheet(frames)[:, :, ::-1])
            summary["files"].append(f.name)
    finally:
        dataset.standardize = was
    for std, key in (("state", dataset._name_map.get("state")), ("actions", dataset._name_map.get("actions"))):
        if key in dataset._numeric:
            arr = dataset._numeric[key][s:e].float().numpy()
            f = out / f"episode_{episode:06d}_{std}.png"
            cv2.imwrite(str(f), plot_lines(arr, std)[:, :, ::-1])
            summary["files"].append(f.name)
            summary[f"{std}_range"] = [arr.min(0).tolist(), arr.max(0).tolist()]
    (out / f"episode_{episode:06d}.json").write_text(json.dumps(summary, indent=2))
    return summary


def main(argv=None) -> None:
    from ..configs.default import DatasetConfig, DatasetMixtureConfig
    from ..configs.train import TrainPipelineConfig
    from ..datasets.factory import make_dataset
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--repo-id", default=None, help="dataset name; optional when --root points at a local dataset")
    ap.add_argument("--root", default=None)
    ap.add_argument("--episode", "--episode-index", dest="episode", type=int, nargs="+", default=[0],
                    help="one or several episode indices")
    ap.add_argument("--output", "--output-dir", dest="output", default="outputs/dataset_viz")
    a = ap.parse_args(argv)
    if a.repo_id is None:
        if a.root is None:
            ap.error("give --repo-id, or --root of a local dataset")
        a.repo_id = f"local/{Path(a.root).name}"
    dc = DatasetConfig(repo_id=a.repo_id, root=a.root)
    cfg = TrainPipelineConfig(dataset_mixture=DatasetMixtureConfig(datasets=[dc]))
    ds = make_dataset(dc, cfg)
    known = set(ds.episodes)
    for ep in a.episode:
        if ep not in known:
            ap.error(f"episode {ep} is not in the dataset (it has {len(known)} episodes)")
        print(json.dumps(visualize_episode(ds, ep, a.output), indent=2))


if __name__ == "__main__":
    main()
