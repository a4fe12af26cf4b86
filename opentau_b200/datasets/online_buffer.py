"""FIFO replay buffer on memory-mapped arrays for data collected while training
(reference ``src/opentau/datasets/online_buffer.py:40-442``).

Frames are appended episode by episode into fixed-capacity ``numpy.memmap`` files (one per feature) and overwritten
oldest-first once full.  ``__getitem__`` returns the frame plus, when ``delta_timestamps`` are given, the temporal
neighbours inside the same episode (nearest timestamp within ``tolerance_s``; out-of-episode queries are flagged
``<key>_is_pad``).  ``compute_sampler_weights`` mixes an offline dataset and the buffer at a requested ratio.
"""

from __future__ import annotations

import os
from pathlib import Path
from typing import Any

import numpy as np
import torch

OCCUPANCY = "_occupancy_mask"
NEXT_INDEX = "_next_index"
INDEX, FRAME_INDEX, EPISODE_INDEX, TIMESTAMP = "index", "frame_index", "episode_index", "timestamp"


class OnlineBuffer(torch.utils.data.Dataset):
    def __init__(self, write_dir: str | Path, data_spec: dict[str, dict] | None, buffer_capacity: int | None,
                 fps: float | None = None, delta_timestamps: dict[str, list[float]] | None = None):
        self.set_delta_timestamps(delta_timestamps)
        self._fps = fps
        self.tolerance_s = 1 / fps - 1e-4 if fps is not None else None
        self._buffer_capacity = buffer_capacity
        spec = self._make_data_spec(data_spec, buffer_capacity)
        Path(write_dir).mkdir(parents=True, exist_ok=True)
        self._data: dict[str, np.memmap] = {}
        for k, v in spec.items():
            path = Path(write_dir) / k
            mode = "r+" if path.exists() else "w+"
            self._data[k] = np.memmap(path, dtype=v["dtype"], mode=mode, shape=tuple(v["shape"]))

    @property
    def delta_timestamps(self):
        return self._delta_timestamps

    def set_delta_timestamps(self, value: dict[str, list[float]] | None) -> None:
        self._delta_timestamps = None if value is None else {k: np.array(v) for k, v in value.items()}

    @staticmethod
    def _make_data_spec(data_spec: dict[str, dict], capacity: int) -> dict[str, dict]:
        if any(k.startswith("_") for k in data_spec):
            raise ValueError("data_spec keys should not start with '_'. This prefix is reserved for internal logic.")
        reserved = {INDEX, FRAME_INDEX, EPISODE_INDEX, TIMESTAMP}
        if reserved & set(data_spec):
            raise ValueError(f"data_spec should not contain any of {sorted(reserved)}: they are added automatically")
        out = {NEXT_INDEX: {"dtype": np.dtype("int64"), "shape": ()},
               OCCUPANCY: {"dtype": np.dtype("?"), "shape": (capacity,)},
               INDEX: {"dtype": np.dtype("int64"), "shape": (capacity,)},
               FRAME_INDEX: {"dtype": np.dtype("int64"), "shape": (capacity,)},
               EPISODE_INDEX: {"dtype": np.dtype("int64"), "shape": (capacity,)},
               TIMESTAMP: {"dtype": np.dtype("float64"), "shape": (capacity,)}}
        for k, v in data_spec.items():
            out[k] = {"dtype": np.dtype(v["dtype"]), "shape": (capacity, *v["shape"])}
        return out

    def add_data(self, data: dict[str, np.ndarray]) -> None:
        """Appends whole episodes; ``index`` / ``episode_index`` are shifted to continue the buffer's numbering."""
        missing = set(self.data_keys) - set(data)
        if missing:
            raise ValueError(f"Missing data keys: {missing}")
        n = len(data[self.data_keys[0]])
        if any(len(data[k]) != n for k in self.data_keys):
            raise ValueError("All data items should have the same length")
        if n > self._buffer_capacity:
            raise ValueError("more frames than the buffer can hold")
        data = {k: np.asarray(v).copy() for k, v in data.items()}
        next_index = int(self._data[NEXT_INDEX])
        if data[EPISODE_INDEX][0] != 0 or data[INDEX][0] != 0:
            raise ValueError("new data must number its episodes and frames from 0")
        if self.num_frames > 0:
            last = (next_index - 1) % self._buffer_capacity
            data[EPISODE_INDEX] += self._data[EPISODE_INDEX][last] + 1
            data[INDEX] += self._data[INDEX][last] + 1
        first = min(n, self._buffer_capacity - next_index)
        for k in self.data_keys:
            self._data[k][next_index:next_index + first] = data[k][:first]
            if first < n:
                self._data[k][:n - first] = data[k][first:]
        self._data[OCCUPANCY][next_index:next_index + first] = True
        if first < n:
            self._data[OCCUPANCY][:n - first] = True
        self._data[NEXT_INDEX][()] = (next_index + n) % self._buffer_capacity

    @property
    def data_keys(self) -> list[str]:
        return sorted(k for k in self._data if k not in (OCCUPANCY, NEXT_INDEX))

    @property
    def fps(self):
        return self._fps

    @property
    def num_episodes(self) -> int:
        return len(np.unique(self._data[EPISODE_INDEX][self._data[OCCUPANCY]]))

    @property
    def num_frames(self) -> int:
        return int(np.count_nonzero(self._data[OCCUPANCY]))

    def __len__(self) -> int:
        return self.num_frames

    def get_data_by_key(self, key: str) -> torch.Tensor:
        return torch.from_numpy(np.asarray(self._data[key][self._data[OCCUPANCY]]))

    def __getitem__(self, idx: int) -> dict[str, Any]:
        if idx >= len(self) or idx < -len(self):
            raise IndexError
        occ = np.flatnonzero(self._data[OCCUPANCY])
        row = occ[idx]
        item = {k: np.asarray(v[row]) for k, v in self._data.items() if not k.startswith("_")}
        if self.delta_timestamps is None:
            return {k: torch.from_numpy(np.asarray(v)) for k, v in item.items()}
        ep = item[EPISODE_INDEX]
        ep_rows = np.flatnonzero((self._data[EPISODE_INDEX] == ep) & self._data[OCCUPANCY])
        ep_ts = self._data[TIMESTAMP][ep_rows]
        for key, dts in self.delta_timestamps.items():
            q = item[TIMESTAMP] + dts
            dist = np.abs(q[:, None] - ep_ts[None, :])
            arg = dist.argmin(axis=1)
            is_pad = dist[np.arange(len(q)), arg] > self.tolerance_s
            inside = (q >= ep_ts.min() - self.tolerance_s) & (q <= ep_ts.max() + self.tolerance_s)
            if np.any(is_pad & inside):
                raise ValueError("query timestamps fall between frames of the episode beyond the tolerance "
                                 f"({self.tolerance_s:.4f}s): the data is not sampled at the declared fps")
            item[key] = self._data[key][ep_rows[arg]]
            item[f"{key}_is_pad"] = is_pad
        return {k: torch.from_numpy(np.asarray(v)) for k, v in item.items()}


def compute_sampler_weights(offline_dataset, offline_drop_n_last_frames: int = 0, online_dataset: OnlineBuffer | None = None,
                            online_sampling_ratio: float | None = None, online_drop_n_last_frames: int = 0) -> torch.Tensor:
    """Per-frame sampling weights for ``[offline frames | online frames]`` so that a fraction
    ``online_sampling_ratio`` of samples comes from the buffer; the last frames of every episode can be excluded."""
    n_off = len(offline_dataset) if offline_dataset is not None else 0
    n_on = len(online_dataset) if online_dataset is not None else 0
    if n_off + n_on == 0:
        raise ValueError("at least one of the datasets must hold data")
    if (n_on > 0) != (online_sampling_ratio is not None):
        raise ValueError("`online_sampling_ratio` must be given exactly when an online dataset with data is given")
    ratio = online_sampling_ratio or 0.0

    def mask(ds, n, drop, from_idx, to_idx):
        m = torch.ones(n, dtype=torch.bool)
        if drop > 0:
            for s, e in zip(from_idx, to_idx):
                m[max(int(s), int(e) - drop):int(e)] = False
        return m

    parts = []
    if n_off:
        edi = offline_dataset.episode_data_index
        m = mask(offline_dataset, n_off, offline_drop_n_last_frames, edi["from"], edi["to"]).float()
        parts.append(m / m.sum() * (1 - ratio))
    if n_on:
        eps = online_dataset.get_data_by_key(EPISODE_INDEX)
        bounds = torch.cat([torch.tensor([0]), torch.nonzero(eps[1:] != eps[:-1]).flatten() + 1, torch.tensor([n_on])])
        m = mask(online_dataset, n_on, online_drop_n_last_frames, bounds[:-1], bounds[1:]).float()
        parts.append(m / m.sum() * ratio)
    w = torch.cat(parts)
    return w / w.sum()
