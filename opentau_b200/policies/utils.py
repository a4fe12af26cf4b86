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


# -- policy-level halves of the "train only ..." flags -----------------------------------------------------------
#: Projections on the flow-matching module that face the dataset's state / action spaces.
STATE_ACTION_PROJECTION_ATTRS: tuple[str, ...] = ("state_proj", "action_in_proj", "action_out_proj")
#: Modules on the backbone+expert wrapper that hold the discrete-action (FAST token) representation.
DISCRETE_ACTION_REPRESENTATION_ATTRS: tuple[str, ...] = ("discrete_action_embedding", "da_head")


def _param_ids_of_attrs(module: nn.Module, attrs: tuple[str, ...]) -> set[int]:
    ids: set[int] = set()
    for a in attrs:
        sub = getattr(module, a, None)
        if isinstance(sub, nn.Module):
            ids.update(id(p) for p in sub.parameters())
        elif isinstance(sub, nn.Parameter):
            ids.add(id(sub))
    return ids


def freeze_policy_level_params_for_vision_only(policy_module: nn.Module, with_expert_module: nn.Module) -> None:
    """``train_vision_encoder_only``, outer half: the wrapper has already left exactly the vision tower and its
    projector trainable; every parameter of the enclosing module that is not the wrapper's is frozen here (state /
    action projections, time MLPs, modality embeddings ...), except a video encoder's ``motion_module``, which is part
    of the vision pathway.  Default-deny instead of a list of names, so that a projection added later cannot keep
    training unnoticed (reference ``src/opentau/policies/utils.py:401-440``)."""
    protected = {id(p) for p in with_expert_module.parameters()}
    for name, p in policy_module.named_parameters():
        if id(p) in protected or "motion_module" in name:
            continue
        p.requires_grad = False


def freeze_with_expert_params_for_state_action_representation_only(with_expert_module: nn.Module) -> list[str]:
    """``train_state_action_representation_only``, inner half: everything the wrapper owns is frozen except the
    discrete-action embedding and head.  Returns the names left trainable (empty for policies without a
    discrete-action pathway; reference ``policies/utils.py:550-584``)."""
    keep = _param_ids_of_attrs(with_expert_module, DISCRETE_ACTION_REPRESENTATION_ATTRS)
    left = []
    for name, p in with_expert_module.named_parameters():
        p.requires_grad = id(p) in keep
        if p.requires_grad:
            left.append(name)
    return sorted(left)


def set_with_expert_train_mode_for_state_action_representation_only(with_expert_module: nn.Module, mode: bool) -> None:
    """Under that flag the frozen trunk runs in eval mode (its dropout would only add noise in front of the two
    trainable modules); the discrete-action modules follow ``mode`` (reference ``policies/utils.py:587-615``)."""
    for child in with_expert_module.children():
        child.eval()
    for a in DISCRETE_ACTION_REPRESENTATION_ATTRS:
        sub = getattr(with_expert_module, a, None)
        if isinstance(sub, nn.Module):
            sub.train(mode)


def freeze_policy_level_params_for_state_action_representation_only(policy_module: nn.Module,
                                                                    with_expert_module: nn.Module) -> list[str]:
    """``train_state_action_representation_only``, outer half: of the enclosing module's own parameters only the
    state / action projections stay trainable; time MLPs, modality embeddings and any video-encoder parameters
    (a freshly initialised ``motion_module`` included) are frozen.  Returns the outer names left trainable
    (reference ``policies/utils.py:618-660``)."""
    protected = {id(p) for p in with_expert_module.parameters()}
    keep = _param_ids_of_attrs(policy_module, STATE_ACTION_PROJECTION_ATTRS)
    left = []
    for name, p in policy_module.named_parameters():
        if id(p) in protected:
            continue
        p.requires_grad = id(p) in keep
        if p.requires_grad:
            left.append(name)
    return sorted(left)


def apply_policy_level_freezes(policy_module: nn.Module, with_expert_module: nn.Module, config) -> None:
    """Call once the flow-matching module is fully built (subclasses add projections after their parent's
    constructor)."""
    if getattr(config, "train_vision_encoder_only", False):
        freeze_policy_level_params_for_vision_only(policy_module, with_expert_module)
    if getattr(config, "train_state_action_representation_only", False):
        freeze_policy_level_params_for_state_action_representation_only(policy_module, with_expert_module)
