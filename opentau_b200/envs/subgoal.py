"""Evaluation-time subgoal images for policies trained with ``subgoal{k}`` inputs (pi0.7 low level and its PaliGemma
variant).

Contract (reference ``src/opentau/envs/subgoal.py:57-640``): a generator is built once per evaluation,
``start_episode(prompts, seeds)`` is called at the top of every rollout and pins the choice for each sub-environment,
and ``generator(observation)`` returns ``{"subgoal{k}": (B,3,H,W) in [0,1], "subgoal_is_pad": (B,) False}`` for every
step of that rollout.  Two generators:

* ``LastFrameSubgoalGenerator``: looks the environment's task string up in a LeRobot dataset on disk, draws one
  matching episode per sub-environment and serves that episode's LAST frame from every camera (a deliberately naive
  baseline: a different trajectory's terminus, matched by language only).
* ``GoalFrameSubgoalGenerator``: a directory of pre-rendered goal frames ``<scene>/<camera>.png`` indexed by the
  rollout seed (what the RoboCasa goal-frame harvest produces).

Frames are resized with aspect-preserving padding to the evaluation resolution and cached per (episode, camera).
"""

from __future__ import annotations

import random
import threading
from pathlib import Path
from typing import Any, Protocol

import numpy as np
import torch
from torch import Tensor

from .. import ops


class SubgoalImageGenerator(Protocol):
    def start_episode(self, prompts: list[str], seeds: list[int] | None = None) -> None: ...

    def __call__(self, observation: dict[str, Any]) -> dict[str, Tensor]: ...


def _fit(img: Tensor, resolution: tuple[int, int]) -> Tensor:
    """``(3,H,W)`` in [0,1] -> padded resize to ``resolution = (H, W)``."""
    h, w = resolution
    if tuple(img.shape[-2:]) == (h, w):
        return img
    return ops.resize_with_pad(img[None].float(), w, h, pad_value=0.0)[0]


def _batch_keys(frames_per_cam: dict[int, list[Tensor]], observation: dict[str, Any]) -> dict[str, Tensor]:
    state = observation["state"]
    dtype = state.dtype if state.dtype.is_floating_point else torch.float32
    out = {f"subgoal{k}": torch.stack(v).to(device=state.device, dtype=dtype) for k, v in frames_per_cam.items()}
    out["subgoal_is_pad"] = torch.zeros(state.shape[0], dtype=torch.bool, device=state.device)
    return out


class LastFrameSubgoalGenerator:
    def __init__(self, root: str | Path, repo_id: str = "local/subgoals", resolution: tuple[int, int] = (224, 224),
                 camera_keys: dict[int, str] | None = None, seed: int | None = None):
        from ..datasets.lerobot_dataset import LeRobotDatasetMetadata
        self.meta = LeRobotDatasetMetadata(repo_id, root=root)
        self.repo_id, self.resolution = repo_id, resolution
        cams = self.meta.camera_keys
        self.camera_keys = camera_keys or dict(enumerate(cams))
        self.lang_to_episodes: dict[str, list[int]] = {}
        for ep, rec in self.meta.episodes.items():
            for task in rec.get("tasks", []):
                self.lang_to_episodes.setdefault(task, []).append(int(ep))
        self._rng = random.Random(seed)
        self._local = threading.local()          # async vector envs evaluate from several threads
        self._cache: dict[tuple[int, str], Tensor] = {}

    @property
    def known_languages(self) -> list[str]:
        return sorted(self.lang_to_episodes)

    def start_episode(self, prompts: list[str], seeds: list[int] | None = None) -> None:
        chosen = []
        for p in prompts:
            cands = self.lang_to_episodes.get(p)
            if not cands:
                raise ValueError(f"no episode of {self.repo_id!r} matches prompt {p!r} "
                                 f"({len(self.lang_to_episodes)} task strings known)")
            chosen.append(self._rng.choice(cands))
        self._local.chosen = chosen

    def _last_frame(self, ep: int, key: str) -> Tensor:
        if (ep, key) not in self._cache:
            length = int(self.meta.episodes[ep]["length"])
            if self.meta.features[key]["dtype"] == "video":
                from ..scripts.annotate_subtasks import frames_at_indices
                got = frames_at_indices(self.meta.root / self.meta.get_video_file_path(ep, key), [length - 1], 10**9)
                if length - 1 not in got:
                    raise RuntimeError(f"could not decode the last frame of episode {ep} / {key}")
                img = np.asarray(got[length - 1])
            else:
                import io

                import pyarrow.parquet as pq
                from PIL import Image
                cell = pq.read_table(self.meta.root / self.meta.get_data_file_path(ep), columns=[key]).column(key)[length - 1].as_py()
                raw = cell.get("bytes") if isinstance(cell, dict) else None
                img = np.asarray((Image.open(io.BytesIO(raw)) if raw else Image.open(self.meta.root / cell["path"])).convert("RGB"))
            t = torch.from_numpy(np.array(img, copy=True)).permute(2, 0, 1).float() / 255.0
            self._cache[(ep, key)] = _fit(t, self.resolution)
        return self._cache[(ep, key)]

    def __call__(self, observation: dict[str, Any]) -> dict[str, Tensor]:
        chosen = getattr(self._local, "chosen", None)
        if chosen is None:
            raise RuntimeError("start_episode(prompts) must be called before the generator is used")
        if observation["state"].shape[0] != len(chosen):
            raise ValueError(f"observation batch {observation['state'].shape[0]} != {len(chosen)} episodes chosen at "
                             "start_episode()")
        return _batch_keys({k: [self._last_frame(ep, key) for ep in chosen] for k, key in self.camera_keys.items()},
                           observation)


class GoalFrameSubgoalGenerator:
    """``root/<scene>/<camera index>.png``; sub-environment ``i`` of a rollout uses scene ``seeds[i] % num_scenes``
    (scene order = sorted directory names)."""

    def __init__(self, root: str | Path, resolution: tuple[int, int] = (224, 224), num_cameras: int | None = None):
        self.root, self.resolution = Path(root), resolution
        self.scenes = sorted(p for p in self.root.iterdir() if p.is_dir())
        if not self.scenes:
            raise FileNotFoundError(f"no scene directory under {self.root}")
        self.num_cameras = num_cameras or len(list(self.scenes[0].glob("*.png")))
        self._local = threading.local()
        self._cache: dict[Path, Tensor] = {}

    @property
    def num_scenes(self) -> int:
        return len(self.scenes)

    def start_episode(self, prompts: list[str], seeds: list[int] | None = None) -> None:
        if seeds is None:
            raise ValueError("goal frames are indexed by the rollout seed: pass seeds")
        self._local.chosen = [self.scenes[int(s) % len(self.scenes)] for s in seeds]

    def _frame(self, path: Path) -> Tensor:
        if path not in self._cache:
            from PIL import Image
            t = torch.from_numpy(np.asarray(Image.open(path).convert("RGB")).copy()).permute(2, 0, 1).float() / 255.0
            self._cache[path] = _fit(t, self.resolution)
        return self._cache[path]

    def __call__(self, observation: dict[str, Any]) -> dict[str, Tensor]:
        chosen = getattr(self._local, "chosen", None)
        if chosen is None:
            raise RuntimeError("start_episode(prompts, seeds) must be called before the generator is used")
        return _batch_keys({k: [self._frame(scene / f"{k}.png") for scene in chosen] for k in range(self.num_cameras)},
                           observation)
