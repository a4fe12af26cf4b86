"""Procedural VQA data for tests and smoke runs (reference ``src/opentau/datasets/vqa/dummy.py``): a coloured square
on a noisy background; the question asks for its colour, or (grounding) for its box in ``<loc>`` tokens."""

from __future__ import annotations

import torch

from ..grounding.loc_codec import xyxy_to_loc_tokens
from .base import VQADataset, register_vqa_dataset

_COLOURS = {"red": (1.0, 0.1, 0.1), "green": (0.1, 1.0, 0.1), "blue": (0.1, 0.1, 1.0), "yellow": (1.0, 1.0, 0.1)}


@register_vqa_dataset("dummy")
class DummyVQADataset(VQADataset):
    def __init__(self, cfg, length: int = 256, grounding: bool = False, train: bool = True):
        self.length, self.grounding = length, grounding
        super().__init__(cfg, train=train)

    def __len__(self) -> int:
        return self.length

    def __getitem_helper__(self, item: int) -> dict:
        g = torch.Generator().manual_seed(item)
        H, W = 96, 128
        img = torch.rand(3, H, W, generator=g) * 0.2
        name = list(_COLOURS)[item % len(_COLOURS)]
        y0 = int(torch.randint(0, H - 32, (1,), generator=g))
        x0 = int(torch.randint(0, W - 32, (1,), generator=g))
        img[:, y0:y0 + 32, x0:x0 + 32] = torch.tensor(_COLOURS[name])[:, None, None]
        if self.grounding:
            return {"image": img, "prompt": "detect square",
                    "postfix": xyxy_to_loc_tokens([(x0, y0, x0 + 32, y0 + 32)], ["square"], (W, H))}
        return {"image": img, "prompt": "what colour is the square?", "postfix": name}
