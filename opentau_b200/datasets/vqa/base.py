"""Vision-language (VQA / grounding) co-training datasets in the standard data format
(reference ``src/opentau/datasets/vqa/base.py:40-200``).

A VQA sample has an image, a question (the ``prompt``) and an answer (the ``response``); it carries a zero state,
a zero action chunk whose ``action_is_pad`` is all True, and therefore trains only the language heads.
"""

from __future__ import annotations

from abc import abstractmethod
from typing import Callable, final

import numpy as np
import torch

from ..lerobot_dataset import BaseDataset

VQA_REGISTRY: dict[str, Callable] = {}


def register_vqa_dataset(name: str):
    def deco(cls):
        VQA_REGISTRY[name] = cls
        return cls
    return deco


def make_vqa_dataset(name: str, cfg, **kw):
    if name not in VQA_REGISTRY:
        raise ValueError(f"unknown vqa dataset {name!r}; registered: {sorted(VQA_REGISTRY)}")
    return VQA_REGISTRY[name](cfg, **kw)


class VQADatasetMetadata:
    def __init__(self, info: dict, stats: dict, repo_id: str):
        self.info, self.stats, self.repo_id = info, stats, repo_id
        self.robot_type, self.control_mode = None, None

    @property
    def features(self) -> dict:
        return self.info["features"]

    @property
    def camera_keys(self) -> list[str]:
        return ["camera0"]


class VQADataset(BaseDataset):
    is_vqa = True        # emits no action chunk: exempt from the mixture's all-delta / all-absolute rule

    def __init__(self, cfg, train: bool = True):
        super().__init__(cfg, name_map={"camera0": "image", "prompt": "prompt", "response": "postfix",
                                        "state": "state", "actions": "actions"}, train=train)
        self.meta = self._make_meta()

    @property
    def num_frames(self) -> int:
        return len(self)

    @property
    def num_episodes(self) -> int:
        return 1

    @property
    def stats(self) -> dict:
        return self.meta.stats

    def _make_meta(self) -> VQADatasetMetadata:
        z = lambda n: np.zeros(n, np.float32)  # noqa: E731
        info = {"features": {"camera0": {"dtype": "image", "shape": (3, *self.resolution), "names": ["channel", "height", "width"]},
                             "state": {"dtype": "float32", "shape": (self.max_state_dim,), "names": None},
                             "actions": {"dtype": "float32", "shape": (self.max_action_dim,), "names": None}}}
        n = np.array([max(1, len(self))])
        stats = {k: {"min": z(d), "max": z(d), "mean": z(d), "std": z(d), "count": n}
                 for k, d in (("state", self.max_state_dim), ("actions", self.max_action_dim))}
        return VQADatasetMetadata(info, stats, self._get_feature_mapping_key())

    @abstractmethod
    def __getitem_helper__(self, item: int) -> dict:
        """Returns ``{"image": (3,H,W) float [0,1], "prompt": str, "postfix": str}``."""

    @final
    def __getitem__(self, item: int) -> dict:
        raw = self.__getitem_helper__(int(item))
        raw["state"] = torch.zeros(self.max_state_dim)
        raw["actions"] = torch.zeros(self.action_chunk, self.max_action_dim)
        raw["actions_is_pad"] = torch.ones(self.action_chunk, dtype=torch.bool)
        out = self._to_standard_data_format(raw)
        out["return_bin_idx"] = torch.tensor(0, dtype=torch.long)
        out["return_continuous"] = torch.tensor(0, dtype=torch.float32)
        out["advantage"] = torch.tensor(0, dtype=torch.bfloat16)
        return out
