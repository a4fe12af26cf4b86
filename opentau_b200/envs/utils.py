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


def add_eval_metadata(observation: dict[str, Any], env_cfg) -> dict[str, Any]:
    """Writes ``env_cfg.metadata`` into an inference batch with the dtypes the dataset emits in training: ``speed`` /
    ``quality`` long and ``mistake`` bool tensors of the batch size, each with ``<key>_is_pad`` all False;
    ``robot_type`` / ``control_mode`` as one string per environment; ``fps`` (the environment's stepping frequency)
    when ``emit_fps`` is set.  Fields that are ``None`` add nothing, so the policy's pad path leaves that segment out
    (reference ``src/opentau/envs/utils.py:234-290``)."""
    meta = getattr(env_cfg, "metadata", None)
    if meta is None:
        return observation
    state = observation["state"]
    n, dev = state.shape[0], state.device
    for key, dtype in (("speed", torch.long), ("quality", torch.long), ("mistake", torch.bool)):
        val = getattr(meta, key)
        if val is not None:
            observation[key] = torch.full((n,), val, dtype=dtype, device=dev)
            observation[f"{key}_is_pad"] = torch.zeros(n, dtype=torch.bool, device=dev)
    for key in ("robot_type", "control_mode"):
        val = getattr(meta, key)
        if val is not None:
            observation[key] = [val] * n
    if meta.emit_fps:
        observation["fps"] = torch.full((n,), int(env_cfg.fps), dtype=torch.long, device=dev)
        observation["fps_is_pad"] = torch.zeros(n, dtype=torch.bool, device=dev)
    return observation


def close_envs(obj) -> None:
    """Closes one environment, or every environment of a (nested) list / dict of them; an environment that fails to
    close is reported and the others are still closed."""
    from collections.abc import Mapping, Sequence
    if obj is None or isinstance(obj, (str, bytes)):
        return
    if isinstance(obj, Mapping):
        for v in obj.values():
            close_envs(v)
    elif isinstance(obj, Sequence):
        for v in obj:
            close_envs(v)
    elif hasattr(obj, "close"):
        try:
            obj.close()
        except Exception as exc:  # noqa: BLE001
            import logging
            logging.warning("exception while closing environment %r: %s", obj, exc)
    else:
        raise NotImplementedError(f"close_envs cannot close a {type(obj).__name__}")


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
