"""VQA corpora read from local files (CLEVR, COCO-QA and VSR in the reference are streamed from the hub:
``src/opentau/datasets/vqa/{clevr,cocoqa,vsr}.py``; there is no network here, so each takes a directory).

Layout: ``<root>/annotations.jsonl`` with rows ``{"image": "relative/path.jpg", "question": str, "answer": str}``
(VSR rows may instead carry ``"caption"`` and ``"label"``: the question becomes *"Is it true that <caption>?"*).
"""

from __future__ import annotations

import json
import os
from pathlib import Path

import numpy as np
import torch

from .base import VQADataset, register_vqa_dataset


class _LocalVQA(VQADataset):
    env_var = "OPENTAU_VQA_ROOT"
    subdir = ""

    def __init__(self, cfg, root: str | None = None, train: bool = True):
        base = root or os.path.join(os.environ.get(self.env_var, ""), self.subdir)
        self.root = Path(base)
        ann = self.root / "annotations.jsonl"
        if not ann.exists():
            raise FileNotFoundError(f"{type(self).__name__}: {ann} not found (set {self.env_var} or pass root)")
        self.rows = [json.loads(line) for line in ann.read_text().splitlines() if line.strip()]
        super().__init__(cfg, train=train)

    def __len__(self) -> int:
        return len(self.rows)

    def _qa(self, row: dict) -> tuple[str, str]:
        return row["question"], str(row["answer"])

    def __getitem_helper__(self, item: int) -> dict:
        from PIL import Image
        row = self.rows[item]
        arr = np.asarray(Image.open(self.root / row["image"]).convert("RGB"))
        q, a = self._qa(row)
        return {"image": torch.from_numpy(arr).permute(2, 0, 1).float() / 255.0, "prompt": q, "postfix": a}


@register_vqa_dataset("clevr")
class CLEVRDataset(_LocalVQA):
    subdir = "clevr"


@register_vqa_dataset("cocoqa")
class COCOQADataset(_LocalVQA):
    subdir = "cocoqa"


@register_vqa_dataset("vsr")
class VSRDataset(_LocalVQA):
    subdir = "vsr"

    def _qa(self, row: dict) -> tuple[str, str]:
        if "caption" in row:
            return f"Is it true that {row['caption'].rstrip('.').lower()}?", "yes" if int(row["label"]) else "no"
        return super()._qa(row)
