"""Image preparation helpers (reference ``src/opentau/utils/vision_utils.py:44-131``): resize keeping the aspect
ratio with padding, and padding to a multiple of the vision patch size.  On CUDA ``resize_with_pad`` is one
hand-written kernel (bilinear sample + pad + scale)."""

from __future__ import annotations

import torch
from torch import Tensor

from .. import ops


def resize_with_pad(img: Tensor, width: int, height: int, pad_value: float = -1.0) -> Tensor:
    if img.dim() != 4:
        raise ValueError(f"(b,c,h,w) expected, but {tuple(img.shape)}")
    return ops.resize_with_pad(img, width, height, pad_value)


def pad_to_patch_multiple(img: Tensor, patch: int, pad_value: float = 0.0) -> Tensor:
    h, w = img.shape[-2:]
    ph, pw = (-h) % patch, (-w) % patch
    if ph == 0 and pw == 0:
        return img
    return torch.nn.functional.pad(img, (0, pw, 0, ph), value=pad_value)
