"""Image augmentations (reference ``src/opentau/datasets/transforms.py:30-330``): a weighted random subset of
colour / sharpness jitters applied in fixed or random order.  Implemented on plain tensors (``(C,H,W)`` in [0,1]) so
no torchvision is needed."""

from __future__ import annotations

import torch
from torch import Tensor

from ..configs.default import ImageTransformsConfig


def _gray(img: Tensor) -> Tensor:
    r, g, b = img.unbind(-3)
    return (0.2989 * r + 0.587 * g + 0.114 * b).unsqueeze(-3)


def _blend(a: Tensor, b: Tensor, ratio: float) -> Tensor:
    return (ratio * a + (1.0 - ratio) * b).clamp(0.0, 1.0)


def adjust_brightness(img: Tensor, f: float) -> Tensor:
    return _blend(img, torch.zeros_like(img), f)


def adjust_contrast(img: Tensor, f: float) -> Tensor:
    return _blend(img, _gray(img).mean(dim=(-3, -2, -1), keepdim=True), f)


def adjust_saturation(img: Tensor, f: float) -> Tensor:
    return _blend(img, _gray(img), f)


def adjust_hue(img: Tensor, f: float) -> Tensor:
    """Rotates the hue by ``f`` (fraction of the colour wheel, in [-0.5, 0.5]) through the YIQ colour space."""
    import math
    th = 2 * math.pi * f
    c, s = math.cos(th), math.sin(th)
    t_yiq = torch.tensor([[0.299, 0.587, 0.114], [0.596, -0.274, -0.322], [0.211, -0.523, 0.312]], dtype=img.dtype)
    rot = torch.tensor([[1, 0, 0], [0, c, -s], [0, s, c]], dtype=img.dtype)
    m = torch.linalg.inv(t_yiq) @ rot @ t_yiq
    return torch.einsum("ij,...jhw->...ihw", m.to(img.device), img).clamp(0.0, 1.0)


def adjust_sharpness(img: Tensor, f: float) -> Tensor:
    k = torch.tensor([[1, 1, 1], [1, 5, 1], [1, 1, 1]], dtype=img.dtype, device=img.device) / 13.0
    x = img.unsqueeze(0) if img.dim() == 3 else img
    C = x.shape[1]
    blur = torch.nn.functional.conv2d(x, k.expand(C, 1, 3, 3), padding=1, groups=C)
    blur[..., 0, :], blur[..., -1, :], blur[..., :, 0], blur[..., :, -1] = x[..., 0, :], x[..., -1, :], x[..., :, 0], x[..., :, -1]
    out = _blend(x, blur, f)
    return out[0] if img.dim() == 3 else out


class RangeJitter:
    def __init__(self, fn, lo: float, hi: float):
        self.fn, self.lo, self.hi = fn, float(lo), float(hi)

    def __call__(self, img: Tensor, generator: torch.Generator | None = None) -> Tensor:
        f = self.lo + (self.hi - self.lo) * float(torch.rand((), generator=generator))
        return self.fn(img, f)


class SharpnessJitter(RangeJitter):
    def __init__(self, sharpness: float | tuple[float, float]):
        if isinstance(sharpness, (int, float)):
            if sharpness < 0:
                raise ValueError("If sharpness is a single number, it must be non negative.")
            sharpness = (max(0.0, 1.0 - sharpness), 1.0 + sharpness)
        lo, hi = sharpness
        if not 0.0 <= lo <= hi:
            raise ValueError(f"sharpness values should be between (0., inf), but got {sharpness}.")
        super().__init__(adjust_sharpness, lo, hi)


def make_transform_from_config(cfg) -> object:
    kw = dict(cfg.kwargs)
    if cfg.type == "Identity":
        return lambda img, generator=None: img
    if cfg.type == "ColorJitter":
        (name, rng), = kw.items()
        fn = {"brightness": adjust_brightness, "contrast": adjust_contrast, "saturation": adjust_saturation,
              "hue": adjust_hue}[name]
        return RangeJitter(fn, *rng)
    if cfg.type == "SharpnessJitter":
        return SharpnessJitter(**kw)
    raise ValueError(f"Transform '{cfg.type}' is not valid.")


class RandomSubsetApply:
    def __init__(self, transforms: list, p: list[float] | None = None, n_subset: int | None = None,
                 random_order: bool = False):
        if p is None:
            p = [1.0] * len(transforms)
        if len(p) != len(transforms):
            raise ValueError("length of p does not match the number of transforms")
        if n_subset is None:
            n_subset = len(transforms)
        if not 1 <= n_subset <= max(1, len(transforms)):
            raise ValueError(f"n_subset should be in the interval [1, {len(transforms)}]")
        tot = sum(p)
        self.transforms, self.p = transforms, [x / tot for x in p]
        self.n_subset, self.random_order = n_subset, random_order

    def __call__(self, img: Tensor, generator: torch.Generator | None = None) -> Tensor:
        idx = torch.multinomial(torch.tensor(self.p), self.n_subset, generator=generator)
        if not self.random_order:
            idx = idx.sort().values
        for i in idx.tolist():
            img = self.transforms[i](img, generator)
        return img


class ImageTransforms:
    def __init__(self, cfg: ImageTransformsConfig):
        self.cfg = cfg
        self.weights, self.transforms = [], {}
        for name, tf in cfg.tfs.items():
            if tf.weight <= 0.0:
                continue
            self.transforms[name] = make_transform_from_config(tf)
            self.weights.append(tf.weight)
        n = min(len(self.transforms), cfg.max_num_transforms)
        self.tf = (RandomSubsetApply(list(self.transforms.values()), self.weights, n, cfg.random_order)
                   if n > 0 and cfg.enable else None)

    def __call__(self, img: Tensor, generator: torch.Generator | None = None) -> Tensor:
        return img if self.tf is None else self.tf(img.float(), generator)
