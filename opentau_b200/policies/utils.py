"""Small helpers shared by the policies (reference ``src/opentau/policies/utils.py:65-385``)."""

from __future__ import annotations

from collections import deque
from typing import NamedTuple

import torch
from torch import Tensor, nn


class PerSampleLoss(NamedTuple):
    """``(sum, count)`` per sample, both ``(B,)``: the summed unmasked loss and the number of slots behind it.

    The masked mean of any group of samples is ``sum.sum() / count.sum()``; carrying the pair instead of a
    per-sample mean lets validation regroup samples by dataset / control mode without double normalising.
    Unpacks like the plain 2-tuple the models return; ``+`` pools two components.
    """

    sum: Tensor
    count: Tensor

    def __add__(self, other):  # type: ignore[override]
        return PerSampleLoss(self.sum + other[0], self.count + other[1])


def ce_per_sample(masked_ce: Tensor, valid_mask: Tensor) -> PerSampleLoss:
    """``masked_ce (B,L)`` already multiplied by its mask -> per-sample sum and slot count."""
    return PerSampleLoss(masked_ce.float().sum(1), valid_mask.to(torch.float32).sum(1))


def make_action_dim_mask(real_action_dim: Tensor | None, max_action_dim: int, batch_size: int, device) -> Tensor:
    """``(B, max_action_dim)`` bool: True on a sample's real action dims, False on zero padding."""
    if real_action_dim is None:
        return torch.ones(batch_size, max_action_dim, dtype=torch.bool, device=device)
    r = torch.as_tensor(real_action_dim, device=device).view(-1, 1)
    return torch.arange(max_action_dim, device=device)[None, :] < r


def populate_queues(queues: dict[str, deque], batch: dict[str, Tensor], exclude_keys: list[str] | None = None):
    """Pushes the newest observation into each rolling queue; a fresh queue is filled by repetition."""
    exclude_keys = exclude_keys or []
    for key in batch:
        if key not in queues or key in exclude_keys:
            continue
        q = queues[key]
        if len(q) != q.maxlen:
            while len(q) != q.maxlen:
                q.append(batch[key])
        else:
            q.append(batch[key])
    return queues


def get_device_from_parameters(module: nn.Module) -> torch.device:
    return next(iter(module.parameters())).device


def get_dtype_from_parameters(module: nn.Module) -> torch.dtype:
    return next(iter(module.parameters())).dtype


def to_dtype_preserving_siglip_float32(module: nn.Module, dtype: torch.dtype) -> nn.Module:
    """Casts ``module``; the SigLIP patch/position embeddings keep fp32 by their own ``_apply`` override."""
    return module.to(dtype)


def assert_gemma3_input_resolution(input_image_size: tuple[int, int] | None, tower_image_size: int) -> None:
    if input_image_size is None:
        return
    if tuple(input_image_size) != (tower_image_size, tower_image_size):
        raise ValueError(f"Gemma-3 vision tower expects {tower_image_size}x{tower_image_size} images, "
                         f"resize_imgs_with_padding is {tuple(input_image_size)}")


def log_model_loading_keys(missing_keys: list[str], unexpected_keys: list[str]) -> None:
    import logging
    if missing_keys:
        logging.warning("Missing key(s) when loading model: %s", missing_keys)
    if unexpected_keys:
        logging.warning("Unexpected key(s) when loading model: %s", unexpected_keys)
