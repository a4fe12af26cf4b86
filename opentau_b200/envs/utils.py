"""Observation plumbing between vector environments and policies (reference ``src/opentau/envs/utils.py:38-320``)."""

from __future__ import annotations

from typing import Any

import numpy as np
import torch
from torch import Tensor


def preprocess_observation(observations: dict[str, Any], cfg=None) -> dict[str, Tensor]:
    """Vector-env observation -> policy batch: ``pixels/*`` uint8 ``(B,H,W,C)`` become float ``(B,C,H,W)`` in [0,1]
    under ``camera{i}``; ``agent_pos`` becomes ``state`` padded to ``max_state_dim``."""
    out: dict[str, Tensor] = {}
    pix = observations.get("pixels")
    if pix is not None:
        imgs = pix if isinstance(pix, dict) else {"camera0": pix}
        for i, (_, img) in enumerate(sorted(imgs.items())):
            t = torch.from_numpy(np.ascontiguousarray(img))
            if t.dim() != 4 or t.shape[-1] != 3:
                raise ValueError(f"expected channel-last (B,H,W,3) images, got {tuple(t.shape)}")
            if t.dtype != torch.uint8:
                raise ValueError(f"expected uint8 images, got {t.dtype}")
            out[f"camera{i}"] = t.permute(0, 3, 1, 2).float() / 255.0
    if "agent_pos" in observations:
        st = torch.from_numpy(np.asarray(observations["agent_pos"])).float()
        n = getattr(cfg, "max_state_dim", None) if cfg is not None else None
        if n and st.shape[-1] < n:
            st = torch.nn.functional.pad(st, (0, n - st.shape[-1]))
        out["state"] = st
    if "environment_state" in observations:
        out["environment_state"] = torch.from_numpy(np.asarray(observations["environment_state"])).float()
    return out


def add_envs_task(env, observation: dict[str, Any]) -> dict[str, Any]:
    """Adds the language instruction of every sub-environment as ``prompt``."""
    n = next(v.shape[0] for v in observation.values() if isinstance(v, Tensor))
    try:
        tasks = list(env.call("task_description"))
    except (AttributeError, TypeError):
        try:
            tasks = list(env.call("task"))
        except (AttributeError, TypeError):
            tasks = [""] * n
    observation["prompt"] = [str(t) for t in tasks]
    return observation


def add_subgoal_images(observation: dict[str, Any], generator) -> dict[str, Any]:
    """Merges ``subgoal{k}`` / ``subgoal_is_pad`` from a subgoal generator into the observation (no-op for None; the
    policy then falls back to zero subgoals marked as padding).  ``generator.start_episode`` must have run."""
    if generator is not None:
        observation.update(generator(observation))
    return observation


def check_env_attributes_and_types(env) -> None:
    import warnings
    for attr in ("task_description", "task"):
        try:
            env.call(attr)
            return
        except (AttributeError, TypeError):
            continue
    warnings.warn("the environment exposes neither `task_description` nor `task`; prompts will be empty",
                  stacklevel=2)
