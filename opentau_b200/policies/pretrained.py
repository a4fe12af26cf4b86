"""Base class of every policy: loss/inference contract and safetensors persistence.

Contract (OpenTau ``src/opentau/policies/pretrained.py:356-1589``):
``forward(batch) -> {"MSE": ..., "CE": ...}``, ``select_action``, ``sample_actions``, ``reset``,
``get_optim_params``, ``from_pretrained`` / ``save_pretrained`` writing ``config.json`` +
``model.safetensors`` with the reference's state-dict key names.
"""

from __future__ import annotations

import abc
import logging
import os
from pathlib import Path
from typing import Any

import torch
from torch import Tensor, nn

from ..configs.policies import PreTrainedConfig
from ..constants import CONFIG_NAME, SAFETENSORS_SINGLE_FILE

_NORM_PREFIXES = ("normalize_inputs.", "normalize_targets.", "normalize_actions.",
                  "normalize_discrete_actions.", "unnormalize_outputs.")


def strip_normalization_buffers(state: dict[str, Tensor]) -> dict[str, Tensor]:
    """Drops every ``(un)normalize_*.buffer_*`` entry (used with ``skip_normalization_weights``)."""
    return {k: v for k, v in state.items() if not k.startswith(_NORM_PREFIXES)}


class PreTrainedPolicy(nn.Module, abc.ABC):
    config_class: type[PreTrainedConfig] | None = None
    name: str | None = None
    #: state-dict prefixes of learned per-group projections (``PerGroupLinear``) that are duplicated / re-ordered by
    #: group name when a checkpoint with another group set is loaded; empty = the policy has none
    _PER_GROUP_PROJECTION_PREFIXES: tuple[str, ...] = ()
    #: policies whose input layers may be wider than an older checkpoint's set this (pi0: the state / action width)
    _TILE_LINEAR_INPUTS = False

    def __init__(self, config: PreTrainedConfig, *inputs, **kwargs):
        super().__init__()
        if not isinstance(config, PreTrainedConfig):
            raise ValueError(f"config must be a PreTrainedConfig, got {type(config).__name__}")
        self.config = config

    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        if not getattr(cls, "config_class", None):
            raise TypeError(f"Class {cls.__name__} must define 'config_class'")
        if not getattr(cls, "name", None):
            raise TypeError(f"Class {cls.__name__} must define 'name'")

    # -- contract ----------------------------------------------------------------------------------
    @abc.abstractmethod
    def get_optim_params(self): ...

    @abc.abstractmethod
    def reset(self): ...

    @abc.abstractmethod
    def forward(self, batch: dict[str, Tensor]) -> dict[str, Tensor]: ...

    @abc.abstractmethod
    def select_action(self, batch: dict[str, Tensor]) -> Tensor: ...

    def sample_actions(self, batch: dict[str, Tensor], **kw) -> Tensor:
        raise NotImplementedError

    def maybe_compile_for_training(self) -> None:
        """Kept for API compatibility: there is no tracing compiler in this framework."""

    # -- normalization heads -----------------------------------------------------------------------
    def _resolve_dataset_index(self, batch: dict[str, Any], batch_size: int, device) -> Tensor:
        """Row of the stacked statistics for each sample.

        Order of precedence: an explicit ``dataset_index`` tensor; ``dataset_repo_id`` names looked
        up in ``config.dataset_to_norm_index`` / ``config.dataset_names``; a single head -> zeros.
        """
        idx = batch.get("dataset_index")
        if idx is not None:
            return torch.as_tensor(idx, device=device).long().reshape(-1)
        names = batch.get("dataset_repo_id")
        cfg = self.config
        if names is not None:
            table = cfg.dataset_to_norm_index or (
                {n: i for i, n in enumerate(cfg.dataset_names)} if cfg.dataset_names else None)
            if table is not None:
                if isinstance(names, str):
                    names = [names] * batch_size
                try:
                    return torch.tensor([table[n] for n in names], dtype=torch.long, device=device)
                except KeyError as e:
                    raise KeyError(f"dataset {e.args[0]!r} has no normalization head; known: {sorted(table)}") from None
        n_heads = len(cfg.dataset_names) if cfg.dataset_names else 1
        if n_heads > 1:
            raise ValueError("the policy has several normalization heads; the batch must carry "
                             "'dataset_index' or 'dataset_repo_id'")
        return torch.zeros(batch_size, dtype=torch.long, device=device)

    def _inject_stats(self, per_dataset_stats: list[dict], dataset_names: list[str] | None = None) -> None:
        """Overwrites every statistics buffer from ``per_dataset_stats`` (one dict per head)."""
        from .normalize import _StatsModule, _as_f32, resolve_stat_row, stat_names_for_mode, _mode_of
        for mod in self.modules():
            if not isinstance(mod, _StatsModule):
                continue
            for key, ft in mod.features.items():
                mode = _mode_of(mod.norm_map, ft)
                buf = getattr(mod, "buffer_" + key.replace(".", "_"), None)
                if buf is None:
                    continue
                for name in stat_names_for_mode(mode):
                    rows = [_as_f32(resolve_stat_row(st, key, name)).reshape(buf[name].shape[1:])
                            for st in per_dataset_stats]
                    t = torch.stack(rows, 0).to(buf[name].device)
                    buf[name] = nn.Parameter(t, requires_grad=False)
            if dataset_names is not None:
                mod.dataset_names = list(dataset_names)
        if dataset_names is not None:
            self.config.dataset_names = list(dataset_names)

    # -- persistence ---------------------------------------------------------------------------------
    def state_dict_for_save(self) -> dict[str, Tensor]:
        state = self.state_dict()
        if not self.config.save_normalization_stats:
            state = strip_normalization_buffers(state)
        return state

    def _save_pretrained(self, save_directory: str | Path) -> None:
        from safetensors.torch import save_file
        save_directory = Path(save_directory)
        save_directory.mkdir(parents=True, exist_ok=True)
        self.config._save_pretrained(save_directory)
        state = self.state_dict_for_save()
        seen: dict[int, str] = {}
        out: dict[str, Tensor] = {}
        for k, v in state.items():  # tied tensors are written once (first name wins)
            key = (v.data_ptr(), tuple(v.shape), v.dtype) if v.numel() else (id(v),)
            if key in seen:
                continue
            seen[key] = k
            out[k] = v.detach().contiguous().cpu()
        save_file(out, str(save_directory / SAFETENSORS_SINGLE_FILE), metadata={"format": "pt"})

    def save_pretrained(self, save_directory: str | Path) -> None:
        self._save_pretrained(save_directory)

    @classmethod
    def from_pretrained(cls, pretrained_name_or_path: str | Path, *, config: PreTrainedConfig | None = None,
                        strict: bool = False, map_location: str = "cpu", **kwargs):
        """``pretrained_name_or_path``: a checkpoint directory or ``repo[@revision]`` in the local cache.  The
        normalisation convention is taken from the checkpoint (``loading.resolve_checkpoint_provenance``) BEFORE
        the policy is built; a local directory without ``model.safetensors`` (a sharded training checkpoint whose
        weights arrive with the optimizer state) yields the constructed policy with a warning, every other missing
        source raises."""
        from . import loading
        if config is None:
            config = PreTrainedConfig.from_pretrained(pretrained_name_or_path)
        loading.resolve_checkpoint_provenance(config, pretrained_name_or_path)
        policy = cls(config, **kwargs)
        try:
            weights = loading.resolve_pretrained_weights_file(pretrained_name_or_path)
        except loading.CheckpointWeightsNotFoundError as exc:
            logging.warning("%s  The policy keeps its initial weights until the training state is loaded.", exc)
            return policy
        old_names = None
        try:
            old_names = PreTrainedConfig.from_pretrained(pretrained_name_or_path).dataset_names
        except Exception:                                          # a checkpoint without a readable config
            pass
        policy = cls._load_as_safetensor(policy, str(weights), map_location, strict, old_dataset_names=old_names)
        policy.eval()
        return policy

    @classmethod
    def _fix_state_dict_keys(cls, state: dict[str, Tensor], config) -> dict[str, Tensor]:
        return state

    @classmethod
    def _load_as_safetensor(cls, model: "PreTrainedPolicy", model_file: str, map_location: str, strict: bool,
                            old_dataset_names: list[str] | None = None):
        from safetensors.torch import load_file
        from . import loading
        state = load_file(model_file, device=map_location if map_location != "cpu" else "cpu")
        state = cls._fix_state_dict_keys(state, model.config)
        if model.config.skip_normalization_weights:
            state = strip_normalization_buffers(state)
            model.config.skip_normalization_weights = False       # one shot: a later save / resume keeps the new stats
        loading.remap_per_group_projection_weights(model, state, cls._PER_GROUP_PROJECTION_PREFIXES, old_dataset_names)
        if cls._TILE_LINEAR_INPUTS:
            loading.tile_linear_input_weights(model, state)
        own = model.state_dict()
        for k, v in list(state.items()):  # linear input tiling / shape guards are policy specific
            if k in own and tuple(own[k].shape) != tuple(v.shape) and k.startswith(_NORM_PREFIXES):
                # legacy (unstacked) statistics: promote to one head
                if tuple(own[k].shape[1:]) == tuple(v.shape):
                    state[k] = v.unsqueeze(0).expand_as(own[k]).clone()
        missing, unexpected = model.load_state_dict(state, strict=False)
        tied = {"model.paligemma_with_expert.paligemma.lm_head.weight"}
        missing = [m for m in missing if m not in tied]
        if missing:
            logging.info("Missing keys when loading state dict: %d keys\n%s", len(missing),
                         "\n".join(f"  - {k}" for k in missing))
        if unexpected:
            logging.info("Unexpected keys when loading state dict: %d keys\n%s", len(unexpected),
                         "\n".join(f"  - {k}" for k in unexpected))
        if strict and (missing or unexpected):
            raise RuntimeError(f"strict load failed: missing={missing} unexpected={unexpected}")
        return model
