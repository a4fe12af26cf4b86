"""Checkpoint-loading behaviours shared by every policy.

What a policy needs between "a name on the command line" and ``load_state_dict`` (reference
``src/opentau/policies/pretrained.py``):

* :func:`peek_config_version` / :func:`resolve_checkpoint_provenance` (``:100-208``): the normalisation convention
  (``config_version``) belongs to the WEIGHTS, not to the code that loads them.  It is read from the checkpoint's
  ``config.json``, else ``train_config.json``, else ``hf_config.json``; a source that carries none is a
  pre-versioning checkpoint (0); a value already set on the config (an explicit override) is kept.  It has to happen
  before the policy is constructed, because the normalisation modules are built from it.
* :func:`resolve_pretrained_weights_file` (``:226-291``): the one place that turns ``dir`` or ``repo[@revision]``
  into ``model.safetensors``; a local directory without weights is its own error class (the shape of a sharded
  optimizer checkpoint that has not been consolidated yet), everything else is ``FileNotFoundError`` with the cause.
* :func:`reconcile_projection_tensor` / :func:`remap_per_group_projection_weights` (``:1088-1210``): learned
  per-group projections (one row per robot / control mode) are duplicated or re-ordered BY GROUP NAME when the
  checkpoint's group set differs from the policy's; a per-group checkpoint never collapses silently into a shared
  projection.
* :func:`tile_linear_input_weights` (``:1389-1416``): a linear layer whose input grew (e.g. a wider state vector)
  takes the checkpoint's columns repeated cyclically.

There is no network here: a ``repo[@revision]`` resolves against the local cache laid out as
``<cache>/<repo>[/<revision>]``.
"""

from __future__ import annotations

import json
import logging
import os
from pathlib import Path

import torch
from torch import Tensor, nn

from ..constants import CONFIG_NAME, SAFETENSORS_SINGLE_FILE, TRAIN_CONFIG_NAME

from ..configs.policies import HF_CONFIG_NAME  # noqa: E402


class CheckpointWeightsNotFoundError(FileNotFoundError):
    """The checkpoint directory exists but holds no ``model.safetensors`` (sharded training state only)."""


class ProjectionRemapError(ValueError):
    """A per-group projection in the checkpoint cannot be mapped onto the policy's groups."""


def _version_in(data: dict) -> int | None:
    """``config_version`` of a policy config, or of the ``policy`` block of a pipeline config."""
    if not isinstance(data, dict):
        return None
    for d in (data, data.get("policy") if isinstance(data.get("policy"), dict) else None):
        if d and isinstance(d.get("config_version"), int):
            return int(d["config_version"])
    return None


def _source_dir(name: str | Path) -> Path | None:
    from ..utils.hub import resolve_local_or_hub
    try:
        p = resolve_local_or_hub(str(name))
    except FileNotFoundError:
        return None
    return p if p.is_dir() else p.parent


def peek_config_version(pretrained_name_or_path: str | Path) -> int | None:
    """Best effort: reads only the version integer, never fails (missing / unreadable -> None)."""
    root = _source_dir(pretrained_name_or_path)
    if root is None:
        return None
    for filename in (CONFIG_NAME, TRAIN_CONFIG_NAME, HF_CONFIG_NAME):
        f = root / filename
        if not f.is_file():
            continue
        try:
            v = _version_in(json.loads(f.read_text()))
        except (OSError, ValueError):
            continue
        if v is not None:
            return v
    return None


def resolve_checkpoint_provenance(config, pretrained_name_or_path: str | Path) -> None:
    """Keys ``config`` (in place) to the conventions its weights were trained under; call right before the policy
    is constructed.  Also warns (never raises) when the stored resize target disagrees with the image features."""
    if config.config_version is None:
        v = peek_config_version(pretrained_name_or_path)
        config.config_version = v if v is not None else 0
    config.validate_input_resolution(strict=False)


def resolve_pretrained_weights_file(pretrained_name_or_path: str | Path) -> str:
    from ..utils.hub import HF_OPENTAU_HOME, split_repo_revision
    name = str(pretrained_name_or_path)
    if os.path.isdir(name):
        f = os.path.join(name, SAFETENSORS_SINGLE_FILE)
        if not os.path.isfile(f):
            raise CheckpointWeightsNotFoundError(
                f"{SAFETENSORS_SINGLE_FILE} not found in local checkpoint directory {name!r}. If this is a sharded "
                "training checkpoint, consolidate it first (python -m opentau_b200.scripts.zero_to_fp32).")
        return f
    if os.path.isfile(name):
        return name
    repo, rev = split_repo_revision(name)
    repo_dir = HF_OPENTAU_HOME / repo
    if not repo_dir.is_dir():
        raise FileNotFoundError(f"repository {repo!r} (from {name!r}) is neither a local path nor in the local cache "
                                f"{HF_OPENTAU_HOME}; this installation does not download")
    from ..utils.hub import cached_revision_dir
    root = cached_revision_dir(repo_dir, rev)
    if rev and not root.is_dir():
        tags = sorted(d.name for d in repo_dir.iterdir() if d.is_dir())
        raise FileNotFoundError(f"revision {rev!r} does not exist in cached repository {repo!r}; training steps are "
                                f"published as tags named by step number.  Cached revisions: {tags or 'none'}.  Omit "
                                "the '@<step>' suffix to load the latest step.")
    f = root / SAFETENSORS_SINGLE_FILE
    if not f.is_file():
        raise FileNotFoundError(f"{SAFETENSORS_SINGLE_FILE} could not be found in {root}")
    return str(f)


ACTION_NORM_META_FILE = "opentau_action_norm.json"


def read_action_norm_meta(tokenizer_path: str | Path) -> dict | None:
    """``{"config_version": int, "zero_range_center": bool}`` stored beside a FAST tokenizer fitted by this framework,
    or ``None`` when the tokenizer is not a local directory / cached snapshot with that file or the file is unreadable:
    a tokenizer without the sidecar (an upstream one, or one fitted before the convention was versioned) makes no
    claim (reference ``src/opentau/policies/pretrained.py:294-331``)."""
    import json
    try:
        root = _source_dir(tokenizer_path)
        if root is None or not (root / ACTION_NORM_META_FILE).is_file():
            return None
        data = json.loads((root / ACTION_NORM_META_FILE).read_text())
    except Exception:  # noqa: BLE001 - best effort by contract
        return None
    return data if isinstance(data, dict) else None


def reconcile_projection_tensor(key: str, loaded: Tensor, target: Tensor, old_names: list[str] | None,
                                new_names: list[str] | None) -> Tensor:
    """The tensor to load for one per-group projection key (``loaded`` itself when nothing has to change)."""
    plain_rank = 2 if key.endswith(".weight") else 1
    if target.ndim != plain_rank + 1:                                   # shared projection in this policy
        if loaded.ndim > target.ndim:
            raise ProjectionRemapError(
                f"{key}: the checkpoint has one projection per group {tuple(loaded.shape)} but this policy shares one "
                f"{tuple(target.shape)}; set per_group_projection=true or load a checkpoint without group heads")
        return loaded
    groups, feat = target.shape[0], tuple(target.shape[1:])
    if loaded.ndim == target.ndim - 1 and tuple(loaded.shape) == feat:   # a single shared layer: one copy per group
        return loaded.unsqueeze(0).expand(groups, *feat).contiguous()
    if loaded.ndim != target.ndim or tuple(loaded.shape[1:]) != feat:
        raise ProjectionRemapError(f"{key}: checkpoint shape {tuple(loaded.shape)} does not fit {tuple(target.shape)}")
    if loaded.shape[0] == 1:
        return loaded.expand(groups, *feat).contiguous()
    if old_names is not None and new_names is not None:
        if list(old_names) == list(new_names):
            return loaded
        at = {n: i for i, n in enumerate(old_names)}
        return torch.stack([loaded[at[n]] if n in at else loaded[0] for n in new_names]).contiguous()
    if loaded.shape[0] == groups:
        return loaded                                                   # same count, nothing known to reorder by
    raise ProjectionRemapError(
        f"{key}: the checkpoint has {loaded.shape[0]} group rows, the policy {groups}, and the checkpoint's group "
        "order is unknown (its config lists no dataset_names)")


def remap_per_group_projection_weights(policy: nn.Module, state: dict[str, Tensor], prefixes: tuple[str, ...],
                                       old_dataset_names: list[str] | None) -> list[str]:
    """In place; returns the keys that were changed.  Only keys under ``prefixes`` are touched."""
    if not prefixes:
        return []
    own = policy.state_dict()
    new_names = getattr(policy.config, "dataset_names", None)
    changed = []
    for key in list(state):
        if not key.startswith(prefixes) or key not in own:
            continue
        t = reconcile_projection_tensor(key, state[key], own[key], old_dataset_names, new_names)
        if t is not state[key]:
            state[key] = t
            changed.append(key)
    if changed:
        logging.info("reconciled %d per-group projection tensor(s) to %s group(s), e.g. %s", len(changed),
                     len(new_names) if new_names else "?", changed[:3])
    return changed


def tile_linear_input_weights(policy: nn.Module, state: dict[str, Tensor]) -> list[str]:
    """In place: every linear layer whose checkpoint weight has fewer input columns than the layer gets the
    checkpoint's columns repeated cyclically up to the layer's width.  Returns the keys that were changed."""
    changed = []
    for name, mod in policy.named_modules():
        w = getattr(mod, "weight", None)
        if not isinstance(mod, nn.Linear) and not (type(mod).__name__ == "Linear" and isinstance(w, Tensor)):
            continue
        key = f"{name}.weight"
        if key not in state or w is None or w.ndim != 2 or state[key].ndim != 2:
            continue
        out_dim, in_dim = state[key].shape
        if w.shape[0] != out_dim:
            raise ValueError(f"{key}: output width {w.shape[0]} differs from the checkpoint's {out_dim}")
        if w.shape[1] == in_dim or w.shape[1] < in_dim:
            continue
        logging.warning("tiling %s from %s to %s input columns", key, in_dim, w.shape[1])
        rep, rem = divmod(w.shape[1], in_dim)
        state[key] = torch.cat([state[key]] * rep + [state[key][:, :rem]], dim=1)
        changed.append(key)
    return changed
