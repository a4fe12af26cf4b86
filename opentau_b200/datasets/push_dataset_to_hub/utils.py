"""Raw-recording helpers used while assembling a dataset for upload (reference
``src/opentau/datasets/push_dataset_to_hub/utils.py:30-131``): episode concatenation with a fresh global index,
threaded PNG dumps, the default video-encoding parameters, repository-id validation and the episode boundaries of a
frame table."""

from __future__ import annotations

import inspect
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Any, Sequence

import numpy as np
import torch


def concatenate_episodes(ep_dicts: Sequence[dict[str, Any]]) -> dict[str, Any]:
    """Tensor columns are concatenated along time, list columns are chained; ``index`` is renumbered from 0."""
    if not ep_dicts:
        raise ValueError("no episodes to concatenate")
    out: dict[str, Any] = {}
    for key in ep_dicts[0]:
        first = ep_dicts[0][key]
        if torch.is_tensor(first) or (len(first) and torch.is_tensor(first[0])):
            out[key] = torch.cat([torch.as_tensor(ep[key]) if torch.is_tensor(ep[key]) else torch.stack(list(ep[key]))
                                  for ep in ep_dicts])
        else:
            out[key] = [x for ep in ep_dicts for x in ep[key]]
    if "frame_index" not in out:
        raise KeyError("episodes need a 'frame_index' column")
    out["index"] = torch.arange(len(out["frame_index"]))
    return out


def save_images_concurrently(imgs_array: np.ndarray, out_dir: str | Path, max_workers: int = 4) -> list[Path]:
    """``frame_000000.png`` ... for every image of ``imgs_array`` (N, H, W, C uint8); returns the paths in order."""
    from PIL import Image
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    paths = [out_dir / f"frame_{i:06d}.png" for i in range(len(imgs_array))]

    def save(i: int) -> None:
        Image.fromarray(np.asarray(imgs_array[i])).save(str(paths[i]))

    with ThreadPoolExecutor(max_workers=max_workers) as pool:
        list(pool.map(save, range(len(paths))))      # list(): a failed write raises here instead of being dropped
    return paths


def get_default_encoding() -> dict:
    """Default encoder parameters of ``video_utils.encode_video_frames`` among vcodec / pix_fmt / g / crf."""
    from ..video_utils import encode_video_frames
    params = inspect.signature(encode_video_frames).parameters
    return {k: v.default for k, v in params.items()
            if v.default is not inspect.Parameter.empty and k in ("vcodec", "pix_fmt", "g", "crf")}


def check_repo_id(repo_id: str) -> None:
    parts = repo_id.split("/")
    if len(parts) != 2 or not all(parts):
        raise ValueError(f"`repo_id` must be '<user or organisation>/<dataset name>' (e.g. 'lerobot/pusht'), "
                         f"got {repo_id!r}")


def calculate_episode_data_index(episode_index: Sequence[int] | Any) -> dict[str, torch.Tensor]:
    """Half-open frame ranges of each run of equal values: ``[0,0,0,1,1,2]`` -> from ``[0,3,5]``, to ``[3,5,6]``.
    Accepts the column itself or a table / mapping with an ``episode_index`` column."""
    if not torch.is_tensor(episode_index) and not isinstance(episode_index, (list, tuple, np.ndarray)):
        episode_index = episode_index["episode_index"]
    ep = torch.as_tensor(np.asarray(episode_index)).long().reshape(-1)
    if ep.numel() == 0:
        return {"from": torch.tensor([]), "to": torch.tensor([])}
    starts = torch.cat([torch.zeros(1, dtype=torch.long), (ep[1:] != ep[:-1]).nonzero().reshape(-1) + 1])
    return {"from": starts, "to": torch.cat([starts[1:], torch.tensor([ep.numel()])])}
