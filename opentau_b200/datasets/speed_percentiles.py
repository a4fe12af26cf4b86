"""Episode speed labels (reference ``src/opentau/datasets/speed_percentiles.py:40-409``): an episode's speed is its
mean per-step state displacement; every episode gets the percentile bucket (1 .. ``n_buckets``) of its speed among
the episodes of the same task, which the pi0.7 metadata block reports as ``"Speed: k"``."""

from __future__ import annotations

import numpy as np


def episode_speed(states: np.ndarray, fps: float) -> float:
    """Mean L2 displacement per second of the state trajectory ``(T, D)``."""
    if len(states) < 2:
        return 0.0
    return float(np.linalg.norm(np.diff(np.asarray(states, np.float64), axis=0), axis=1).mean() * fps)


def speed_buckets(speeds: dict[int, float], tasks: dict[int, str], n_buckets: int = 5) -> dict[int, int]:
    """``episode -> bucket`` with buckets formed per task (ties broken by episode index for determinism)."""
    out: dict[int, int] = {}
    by_task: dict[str, list[int]] = {}
    for ep, t in tasks.items():
        by_task.setdefault(t, []).append(ep)
    for eps in by_task.values():
        order = sorted(eps, key=lambda e: (speeds[e], e))
        for rank, ep in enumerate(order):
            out[ep] = min(n_buckets, int(rank * n_buckets / len(order)) + 1)
    return out


def compute_speed_labels(dataset, n_buckets: int = 5) -> dict[int, int]:
    """Works on a :class:`~opentau_b200.datasets.lerobot_dataset.LeRobotDataset`."""
    key = dataset._name_map.get("state", "observation.state")
    col = dataset._numeric[key].numpy()
    speeds, tasks = {}, {}
    for ep in dataset.episodes:
        i = dataset.epi2idx[ep]
        s, e = int(dataset.episode_data_index["from"][i]), int(dataset.episode_data_index["to"][i])
        speeds[ep] = episode_speed(col[s:e], dataset.fps)
        tasks[ep] = ",".join(dataset.meta.episodes[ep].get("tasks", []))
    return speed_buckets(speeds, tasks, n_buckets)
