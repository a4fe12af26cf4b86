"""Base class of every policy: loss/inference contract and safetensors persistence.

Contract (OpenTau ``src/opentau/policies/pretrained.py:356-1589``):
``forward(batch) -> {"MSE": ..., "CE": ...}``, ``select_action``, ``sample_actions``, ``reset``,
``get_optim_params``, ``from_pretrained`` / ``save_pretrained`` writing ``config.json`` +
``model.safetensors`` with the reference's state-dict key names.
"""

from __future__ import annotations

import abc
import logging
import re
import os
from pathlib import Path
from typing import Any

import torch
from torch import Tensor, nn

from ..configs.policies import PreTrainedConfig
from ..constants import CONFIG_NAME, SAFETENSORS_SINGLE_FILE
from ..utils.hub import HubMixin

_NORM_PREFIXES = ("normalize_inputs.", "normalize_targets.", "normalize_actions.",
                  "normalize_discrete_actions.", "unnormalize_outputs.")


_NORM_BUFFER_KEY = re.compile(r"(^|\.)(un)?normalize_[a-z_]+\.buffer_")


def is_norm_buffer_key(key: str) -> bool:
    """``normalize_*.buffer_*`` / ``unnormalize_*.buffer_*`` at the top level or under a wrapper prefix."""
    return bool(_NORM_BUFFER_KEY.search(key))


def strip_normalization_buffers(state: dict[str, Tensor]) -> dict[str, Tensor]:
    """Drops every ``(un)normalize_*.buffer_*`` entry (used with ``skip_normalization_weights``)."""
    return {k: v for k, v in state.items() if not is_norm_buffer_key(k)}


class PreTrainedPolicy(nn.Module, HubMixin, abc.ABC):
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
    #: batch keys that identify a sample but carry no data (skipped when the batch size / device are inferred)
    _NON_DATA_BATCH_KEYS = frozenset({"dataset_index", "dataset_repo_id", "robot_type", "control_mode"})

    @property
    def _norm_key_to_index(self) -> dict[str, int] | None:
        """``{head key: row}`` from ``config.dataset_names`` (the head keys, one per row); ``None`` = no names."""
        names = self.config.dataset_names
        return {n: i for i, n in enumerate(names)} if names else None

    @property
    def _dataset_to_norm_index(self) -> dict[str, int] | None:
        """``{training dataset name: row}``; a checkpoint that stored only the head keys gets the identity table."""
        table = self.config.dataset_to_norm_index
        return dict(table) if table else self._norm_key_to_index

    def _model_device(self) -> torch.device:
        try:
            return next(self.parameters()).device
        except StopIteration:
            return torch.device("cpu")

    def _stat_modules(self):
        from .normalize import _StatsModule
        return [m for m in self.modules() if isinstance(m, _StatsModule)]

    def _iter_norm_buffer_params(self):
        for mi, mod in enumerate(self._stat_modules()):
            for name, p in mod.named_parameters(recurse=True):
                if name.startswith("buffer_"):
                    yield f"{type(mod).__name__.lower()}[{mi}].{name}", p

    def _stacked_num_datasets(self) -> int:
        """Rows of the stacked statistics, read from the buffers themselves: the one source of truth, also for a policy
        built directly with two statistics dicts and no names.  1 when there is no statistics buffer at all."""
        for _, p in self._iter_norm_buffer_params():
            return int(p.shape[0])
        return 1

    def _norm_buffers_have_inf(self) -> bool:
        """True while any statistics buffer still holds the ``+inf`` it was created with, i.e. was neither loaded from
        a checkpoint nor filled from statistics (a checkpoint saved with ``save_normalization_stats=False``)."""
        return any(bool(torch.isinf(p).any()) for _, p in self._iter_norm_buffer_params())

    def _check_norm_stats_loaded(self) -> None:
        """Fails at construction time, with the buffer names, instead of at the first forward pass."""
        bad = [n for n, p in self._iter_norm_buffer_params() if bool(torch.isinf(p).any())]
        if bad:
            raise RuntimeError("normalisation buffers were neither loaded from the checkpoint nor given statistics; "
                               f"still +inf: {bad}.  Save the checkpoint with `save_normalization_stats=True`, or pass "
                               "`ds_meta=` to `make_policy(...)` so that statistics are injected after the load.")

    def _check_discrete_action_tokenizer_convention(self, tokenizer_path: str | Path) -> None:
        """A fitted FAST tokenizer bakes the zero-range convention of the normalised actions into its BPE corpus
        (version 0: a zero-range dim maps to -1; later: to 0), so tokenizer and policy must agree or padded action
        columns tokenize to values the corpus never saw.  Only tokenizers fitted by this framework carry the sidecar;
        one without it makes no claim and passes (reference ``src/opentau/policies/pretrained.py:996-1044``)."""
        from .loading import read_action_norm_meta
        meta = read_action_norm_meta(tokenizer_path)
        if meta is None or "zero_range_center" not in meta:
            return
        ours = bool(self.config.zero_range_centers_on_zero)
        if bool(meta["zero_range_center"]) != ours:
            v = self.config.resolved_config_version()
            raise ValueError(
                f"FAST tokenizer / policy normalisation mismatch: the tokenizer at '{tokenizer_path}' was fitted with "
                f"zero_range_center={bool(meta['zero_range_center'])} (config_version {meta.get('config_version', '?')}), "
                f"this policy resolves to zero_range_center={ours} (config_version {v}).  Re-fit the tokenizer with "
                f"`fit_fast_tokenizer --config-version {v}`, or pin the policy with "
                f"`--policy.config_version={meta.get('config_version', 0)}`.")

    def _infer_batch_size_and_device(self, batch: dict[str, Any]) -> tuple[int, torch.device]:
        for key, v in batch.items():
            if key not in self._NON_DATA_BATCH_KEYS and isinstance(v, Tensor):
                return (v.shape[0] if v.ndim > 0 else 1), v.device
        return 0, self._model_device()

    def _resolve_dataset_index(self, batch: dict[str, Any], batch_size: int | None = None, device=None) -> Tensor:
        """Row of the stacked statistics for each sample (reference ``src/opentau/policies/pretrained.py:681-829``).

        First match wins:

        1. ``dataset_index``: the tensor the mixture tags every training sample with.  The only route used in training,
           because ``robot_type`` / ``control_mode`` are subject to per-sample dropout there.
        2. ``robot_type`` AND ``control_mode`` (a string or one per sample): looked up as ``"<rt>::<cm>"`` among the
           head keys; a pair that was dropped or is unknown raises instead of picking a row.
        3. ``dataset_repo_id`` (a string or one per sample): training dataset name -> row, which also works when
           several datasets share a head.
        4. nothing of the above and ONE row: zeros.  With several rows the batch must identify itself.

        A single-head policy without name tables (an old checkpoint) answers routes 2 and 3 with row 0: there is
        nothing to resolve.  ``KeyError``: unidentifiable batch on a multi-head policy; ``ValueError``: an identifier
        that matches no row; ``RuntimeError``: names given to a multi-head policy that has no name tables."""
        inferred_b, inferred_dev = self._infer_batch_size_and_device(batch)
        B = batch_size if batch_size is not None else (inferred_b or 1)
        dev = device if device is not None else inferred_dev
        idx = batch.get("dataset_index")
        if idx is not None:
            # onto the device of the statistics, not of whichever batch tensor comes first
            return torch.as_tensor(idx).to(dtype=torch.long, device=device if device is not None
                                           else self._model_device()).reshape(-1)

        def single_head():
            return torch.zeros(B, dtype=torch.long, device=dev) if self._stacked_num_datasets() <= 1 else None

        def spread(v):
            return [v] * B if isinstance(v, str) else list(v)

        if batch.get("robot_type") is not None and batch.get("control_mode") is not None:
            table = self._norm_key_to_index
            if table is None:
                row0 = single_head()
                if row0 is not None:
                    return row0
                raise RuntimeError("the policy has several normalisation heads but no `dataset_names`: it cannot map "
                                   "(robot_type, control_mode) to a head; pass `dataset_index`, or build the policy "
                                   "through `make_policy(cfg, ds_meta=...)`")
            from ..datasets.dataset_mixture import compute_norm_key
            rts, cms = spread(batch["robot_type"]), spread(batch["control_mode"])
            if len(rts) != len(cms):
                raise ValueError(f"`robot_type` ({len(rts)}) and `control_mode` ({len(cms)}) differ in length")
            keys = [compute_norm_key(rt, cm, "")[0] for rt, cm in zip(rts, cms)]     # "" matches no row: raises below
            if not any(k in table for k in keys):
                row0 = single_head()          # one head under another name (a hand-named or name-keyed head)
                if row0 is not None:
                    return row0
            try:
                return torch.tensor([table[k] for k in keys], dtype=torch.long, device=dev)
            except KeyError as e:
                raise ValueError(f"norm key {e.args[0]!r} (from robot_type / control_mode) is not one of this policy's "
                                 f"heads {list(table)}") from None
        names = batch.get("dataset_repo_id")
        if names is not None:
            table = self._dataset_to_norm_index
            if table is None:
                row0 = single_head()
                if row0 is not None:
                    return row0
                raise RuntimeError("the policy has several normalisation heads but no `dataset_names`: it cannot map "
                                   "`dataset_repo_id` to a head; pass `dataset_index`, or build the policy through "
                                   "`make_policy(cfg, ds_meta=...)`")
            try:
                return torch.tensor([table[n] for n in spread(names)], dtype=torch.long, device=dev)
            except KeyError as e:
                row0 = single_head()
                if row0 is not None:
                    return row0
                raise ValueError(f"dataset_repo_id {e.args[0]!r} is not in this policy's training set "
                                 f"{sorted(table)}") from None
        rows = self._stacked_num_datasets()
        if rows <= 1:
            return torch.zeros(B, dtype=torch.long, device=dev)
        raise KeyError(f"normalisation with {rows} heads needs one of `dataset_index` (LongTensor (B,)), "
                       "`dataset_repo_id` (str or one per sample), or both `robot_type` and `control_mode` in the batch")

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
    def _strip_normalization_buffers_from_state_dict(cls, state: dict[str, Tensor], config, *,
                                                     is_main_process: bool = True) -> tuple[dict[str, Tensor], frozenset]:
        """With ``config.skip_normalization_weights`` the statistics stored in the checkpoint are ignored, so that the
        buffers built from the CURRENT mixture survive the load (fine-tuning a checkpoint whose statistics were pooled
        over other data; the buffers do not train, so nothing else would correct them).  Returns the filtered dict and
        the dropped keys.  The flag is consumed by this load whether or not anything was dropped (a later save stores
        ``False``, so a resume does not strip the now-correct buffers); a flag that dropped nothing is reported, since
        the user expected it to void something (reference ``src/opentau/policies/pretrained.py:1213-1305``)."""
        if not config.skip_normalization_weights:
            return state, frozenset()
        dropped = frozenset(k for k in state if is_norm_buffer_key(k))
        config.skip_normalization_weights = False
        if not dropped:
            if is_main_process:
                logging.warning("skip_normalization_weights=True, but the checkpoint holds no normalize_ / unnormalize_ "
                                "keys: the flag had no effect")
            return state, dropped
        if is_main_process:
            logging.info("skip_normalization_weights=True: dropped %d stored statistics buffers", len(dropped))
        return {k: v for k, v in state.items() if k not in dropped}, dropped

    @classmethod
    def _promote_legacy_norm_buffers(cls, model: "PreTrainedPolicy", state: dict[str, Tensor]) -> None:
        """Checkpoints from before the stacked layout store statistics as ``(*feature_shape,)``; the buffers are now
        ``(heads, *feature_shape)``.  A stored tensor exactly one rank short of its buffer becomes the single row of a
        one-head policy (such a checkpoint was trained on one mixture); in place, one warning."""
        own = model.state_dict()
        promoted = []
        for k, v in list(state.items()):
            tgt = own.get(k)
            if tgt is None or not is_norm_buffer_key(k):
                continue
            if v.dim() == tgt.dim() - 1 and tuple(v.shape) == tuple(tgt.shape[1:]):
                state[k] = v.unsqueeze(0).expand_as(tgt).clone()
                promoted.append(k)
        if promoted:
            logging.warning("promoted %d single-dataset statistics buffers to the stacked (heads, ...) layout, e.g. %s",
                            len(promoted), promoted[:3])

    @classmethod
    def _assert_normalize_buffers_initialized(cls, model: "PreTrainedPolicy", *, stripped_keys: frozenset) -> None:
        """After a load that dropped the stored statistics, fresh ones must have been given to the constructor;
        otherwise the first forward pass would fail with a message about "a pretrained model", which misleads when a
        pretrained model WAS used and its statistics were dropped on purpose."""
        if not stripped_keys:
            return
        bad = [n for n, p in model._iter_norm_buffer_params() if bool(torch.isinf(p).any())]
        if bad:
            raise ValueError("skip_normalization_weights=True needs `per_dataset_stats` at construction (e.g. "
                             "`make_policy(..., ds_meta=...)`) to replace the dropped statistics; "
                             f"{len(bad)} buffer(s) are still +inf: " + ", ".join(bad[:5])
                             + (f", ... ({len(bad) - 5} more)" if len(bad) > 5 else ""))

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
        state, stripped = cls._strip_normalization_buffers_from_state_dict(state, model.config)
        loading.remap_per_group_projection_weights(model, state, cls._PER_GROUP_PROJECTION_PREFIXES, old_dataset_names)
        if cls._TILE_LINEAR_INPUTS:
            loading.tile_linear_input_weights(model, state)
        cls._promote_legacy_norm_buffers(model, state)
        missing, unexpected = model.load_state_dict(state, strict=False)
        tied = {"model.paligemma_with_expert.paligemma.lm_head.weight"}
        missing = [m for m in missing if m not in tied and m not in stripped]      # dropped on purpose: not "missing"
        cls._assert_normalize_buffers_initialized(model, stripped_keys=stripped)
        if missing:
            logging.info("Missing keys when loading state dict: %d keys\n%s", len(missing),
                         "\n".join(f"  - {k}" for k in missing))
        if unexpected:
            logging.info("Unexpected keys when loading state dict: %d keys\n%s", len(unexpected),
                         "\n".join(f"  - {k}" for k in unexpected))
        if strict and (missing or unexpected):
            raise RuntimeError(f"strict load failed: missing={missing} unexpected={unexpected}")
        return model
