"""Base policy configuration and the ``type`` registry of policy configs.

Field names, defaults and the ``config.json`` file format follow the reference
(OpenTau ``src/opentau/configs/policies.py:290-476,813-985``); the codec is our own.
"""

from __future__ import annotations

import abc
import json
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, ClassVar

from ..utils.hub import HubMixin
from ..constants import CONFIG_NAME, TRAIN_CONFIG_NAME
from .codec import ChoiceRegistry, decode, encode
from .types import FeatureType, NormalizationMode, PolicyFeature

# Version of the behavioural conventions a checkpoint's weights were trained under (not the package version):
#   0  legacy: a zero-range MIN_MAX / QUANTILE band maps to -1.0, normalisation epsilon 1e-8
#   1  a zero-range band maps to 0.0 and the epsilon is 1e-6
# A config without the field runs as CURRENT in a fresh run and is resolved to 0 when weights that predate the field
# are loaded (policies/loading.py: resolve_checkpoint_provenance).
CURRENT_CONFIG_VERSION = 1
OPENPI_EPS = 1e-6   # normalization epsilon for config_version >= 1
LEGACY_EPS = 1e-8   # epsilon for checkpoints without a version

#: whole-pipeline configs that a checkpoint folder may hold instead of (or beside) ``config.json``; their ``policy``
#: object is a valid policy config, so both config loaders fall back to them
HF_CONFIG_NAME = "hf_config.json"

DEPRECATED_LATENCY_FIELDS = ("cloud_vlm_latency_mean", "cloud_vlm_latency_std", "cloud_vlm_latency_lower",
                             "cloud_vlm_latency_upper", "action_decoder_latency_mean", "action_decoder_latency_std",
                             "action_decoder_latency_lower", "action_decoder_latency_upper")
#: removed from the dataclass: dropped from incoming JSON (old configs still load) and from outgoing JSON
REMOVED_POLICY_FIELDS = ("init_strategy",)
STRIPPED_FIELDS = DEPRECATED_LATENCY_FIELDS + REMOVED_POLICY_FIELDS


def strip_keys(data: dict, keys: tuple[str, ...]) -> bool:
    """Drops ``keys`` at the top level and under a ``"policy"`` object; True if anything changed."""
    changed = False
    for scope in (data, data.get("policy") if isinstance(data.get("policy"), dict) else None):
        if scope is None:
            continue
        for k in keys:
            if k in scope:
                del scope[k]
                changed = True
    return changed


def find_present_keys(data: dict, keys: tuple[str, ...]) -> list[str]:
    found = [k for k in keys if k in data]
    if isinstance(data.get("policy"), dict):
        found += [f"policy.{k}" for k in keys if k in data["policy"]]
    return found


def strip_deprecated_fields_from_json(path: str | Path) -> None:
    """Rewrites a config file WE own (one just written into a save directory) without the stripped fields.  Never
    for incoming files: a hub cache path is a link into a content-addressed store and a rewrite would corrupt it;
    incoming configs are stripped in memory (:func:`stripped_copy`)."""
    data = json.loads(Path(path).read_text())
    if strip_keys(data, STRIPPED_FIELDS):
        Path(path).write_text(json.dumps(data, indent=4))


def load_resolved_config_dict(source_path: str | Path) -> dict:
    """The config as one dict with ``$ref`` includes resolved; a non-object root is an error for every loader."""
    from .refs import load_json_with_refs
    data = load_json_with_refs(source_path)
    if not isinstance(data, dict):
        raise TypeError(f"Top-level config at {source_path} must be a JSON object after $ref resolution, "
                        f"got {type(data).__name__}")
    return data


def stripped_copy(data: dict) -> dict:
    """``data`` without the stripped fields; the caller's dict is left as it was (two-level copy: the keys only
    ever live at the top level or under ``policy``)."""
    out = dict(data)
    if isinstance(out.get("policy"), dict):
        out["policy"] = dict(out["policy"])
    strip_keys(out, STRIPPED_FIELDS)
    return out


def warn_deprecated_latency_fields_from_dict(data: dict, config_path: str | Path) -> None:
    import warnings
    found = find_present_keys(data, DEPRECATED_LATENCY_FIELDS)
    if found:
        warnings.warn(f"Config '{config_path}' contains deprecated latency fields that are no longer used and will "
                      f"be ignored: {', '.join(found)}. Consider re-saving the config to remove them.",
                      DeprecationWarning, stacklevel=4)


def warn_removed_policy_fields_from_dict(data: dict, config_path: str | Path) -> None:
    import warnings
    found = find_present_keys(data, REMOVED_POLICY_FIELDS)
    if found:
        warnings.warn(f"Config '{config_path}' contains fields that have been removed and will be ignored: "
                      f"{', '.join(found)}. Re-save the config to drop them.", DeprecationWarning, stacklevel=4)


def warn_deprecated_latency_fields(config_path: str | Path) -> None:
    """Warns when a config file (``$ref`` includes followed) still carries latency fields."""
    warn_deprecated_latency_fields_from_dict(load_resolved_config_dict(config_path), config_path)


def warn_removed_policy_fields(config_path: str | Path) -> None:
    """Warns when a config file carries a removed field: the user's explicit choice is being dropped."""
    warn_removed_policy_fields_from_dict(load_resolved_config_dict(config_path), config_path)


@dataclass
class PreTrainedConfig(ChoiceRegistry, HubMixin, abc.ABC):
    n_obs_steps: int = 1
    normalization_mapping: dict[str, NormalizationMode] = field(default_factory=dict)
    input_features: dict[str, PolicyFeature] = field(default_factory=dict)
    output_features: dict[str, PolicyFeature] = field(default_factory=dict)
    device: str | None = None
    use_amp: bool = False
    accel_prefix: int | str | None = None
    n_candidates: int = 1
    action_chunk_critic_path: str | None = None
    use_torch_compile: bool = False
    torch_compile_mode: str = "default"
    pretrained_path: str | None = None
    skip_normalization_weights: bool = False
    skip_input_resolution_check: bool = False
    save_normalization_stats: bool = True
    dataset_names: list[str] | None = None
    dataset_to_norm_index: dict[str, int] | None = None
    config_version: int | None = None
    opentau_version: str | None = None
    cloud_vlm_latency_mean: float = 0.0
    cloud_vlm_latency_std: float = 0.0
    cloud_vlm_latency_lower: float = 0.0
    cloud_vlm_latency_upper: float = 0.0
    action_decoder_latency_mean: float = 0.0
    action_decoder_latency_std: float = 0.0
    action_decoder_latency_lower: float = 0.0
    action_decoder_latency_upper: float = 0.0

    action_horizon_delay_field: ClassVar[str] = "max_delay"
    _deprecated_fields: ClassVar[tuple[str, ...]] = ("job_name", "advantage_threshold", "tokenizer_max_length")

    def __post_init__(self):
        if self.device is None:
            try:
                import torch
                self.device = "cuda" if torch.cuda.is_available() else "cpu"
            except Exception:  # pragma: no cover
                self.device = "cpu"
        self.normalization_mapping = {
            (k.value if isinstance(k, FeatureType) else str(k)): NormalizationMode(v)
            for k, v in self.normalization_mapping.items()}

    # -- properties mirroring the reference API ----------------------------------------------------
    @property
    def type(self) -> str:
        return self.get_choice_name()

    def resolved_config_version(self) -> int:
        """The version behaviour reads through: an unresolved ``None`` is a fresh run and runs as CURRENT.  The
        stored field stays ``None`` until a save or the checkpoint-provenance resolution makes it concrete."""
        return self.config_version if self.config_version is not None else CURRENT_CONFIG_VERSION

    @property
    def zero_range_centers_on_zero(self) -> bool:
        """New-format checkpoints map a zero-range dim to 0; legacy ones to -1."""
        return self.resolved_config_version() >= 1

    @property
    def normalization_epsilon(self) -> float:
        return OPENPI_EPS if self.resolved_config_version() >= 1 else LEGACY_EPS

    @property
    def robot_state_feature(self) -> PolicyFeature | None:
        for ft in self.input_features.values():
            if ft.type is FeatureType.STATE:
                return ft
        return None

    @property
    def image_features(self) -> dict[str, PolicyFeature]:
        return {k: ft for k, ft in self.input_features.items() if ft.type is FeatureType.VISUAL}

    @property
    def action_feature(self) -> PolicyFeature | None:
        for ft in self.output_features.values():
            if ft.type is FeatureType.ACTION:
                return ft
        return None

    @property
    def observation_delta_indices(self):
        return None

    @property
    def action_delta_indices(self):
        n = getattr(self, "chunk_size", None)
        return list(range(n)) if n else None

    @property
    def reward_delta_indices(self):
        return None

    def get_optimizer_preset(self):
        from ..optim.optimizers import AdamWConfig
        return AdamWConfig(lr=getattr(self, "optimizer_lr", 2.5e-5),
                           betas=tuple(getattr(self, "optimizer_betas", (0.9, 0.95))),
                           eps=getattr(self, "optimizer_eps", 1e-8),
                           weight_decay=getattr(self, "optimizer_weight_decay", 1e-10))

    def get_scheduler_preset(self):
        from ..optim.schedulers import CosineDecayWithWarmupSchedulerConfig
        return CosineDecayWithWarmupSchedulerConfig(
            peak_lr=getattr(self, "optimizer_lr", 2.5e-5),
            decay_lr=getattr(self, "scheduler_decay_lr", 2.5e-6),
            num_warmup_steps=getattr(self, "scheduler_warmup_steps", 1000),
            num_decay_steps=getattr(self, "scheduler_decay_steps", 30000))

    def validate_features(self) -> None:
        pass

    def validate_action_horizon(self) -> None:
        """``n_action_steps <= chunk_size`` and the real-time delay leaves at least one action."""
        chunk = getattr(self, "chunk_size", None)
        steps = getattr(self, "n_action_steps", None)
        delay = getattr(self, self.action_horizon_delay_field, 0) if self.action_horizon_delay_field else 0
        if chunk is None or steps is None:
            return
        if steps > chunk:
            raise ValueError(f"n_action_steps ({steps}) must be <= chunk_size ({chunk})")
        if delay and delay >= chunk:
            raise ValueError(f"{self.action_horizon_delay_field} ({delay}) must be < chunk_size ({chunk})")

    def _bound_image_resolutions(self) -> dict[str, tuple[int, int]]:
        """``(H, W)`` of every bound visual feature with a ``(C, H, W)`` shape."""
        out = {}
        for key, ft in self.image_features.items():
            shape = tuple(getattr(ft, "shape", ()) or ())
            if len(shape) == 3:
                out[key] = (int(shape[1]), int(shape[2]))
        return out

    @property
    def input_image_size(self) -> tuple[int, int] | None:
        """``(H, W)`` at which frames reach the vision tower: the resize target, or (native pass-through) the one
        resolution the image features were bound at; ``None`` when that is unknown or mixed."""
        target = getattr(self, "resize_imgs_with_padding", None)
        if target is not None:
            return tuple(int(x) for x in target)
        bound = set(self._bound_image_resolutions().values())
        return next(iter(bound)) if len(bound) == 1 else None

    def validate_input_resolution(self, *, strict: bool) -> None:
        """``resize_imgs_with_padding`` must equal the resolution of the bound image features, else every frame is
        letterboxed a second time inside the policy; with ``None`` (native pass-through) all cameras must agree with
        each other.  ``strict`` (training-shaped construction) raises unless ``skip_input_resolution_check``; an
        eval / inference load only warns so that checkpoints trained with the mismatch stay loadable (reference
        ``src/opentau/configs/policies.py:732-799``)."""
        import dataclasses
        if "resize_imgs_with_padding" not in {f.name for f in dataclasses.fields(self)}:
            return                       # no such setting (or a derived one: the policy always resizes to it)
        target = self.resize_imgs_with_padding
        bound = self._bound_image_resolutions()
        if target is None:
            if len(set(bound.values())) <= 1:
                return
            listed = ", ".join(f"{k}={v}" for k, v in sorted(bound.items()))
            msg = (f"resize_imgs_with_padding is null (native pass-through) but the bound image features have mixed "
                   f"resolutions: {listed}; give one (H, W) target instead.")
        else:
            target = tuple(int(x) for x in target)
            off = {k: v for k, v in bound.items() if v != target}
            if not off:
                return
            listed = ", ".join(f"{k}={v}" for k, v in sorted(off.items()))
            msg = (f"resize_imgs_with_padding={target} (H, W) differs from the bound image features: {listed}. The "
                   "policy would resample and pad every frame a second time. Set it to the input resolution, or to "
                   "null to pass frames through (PaliGemma-family policies only).")
        if strict and not self.skip_input_resolution_check:
            raise ValueError(msg + " To resume a checkpoint trained with this mismatch set "
                                   "policy.skip_input_resolution_check=true.")
        import logging
        logging.warning("%s Proceeding because this is %s.", msg,
                        "skip_input_resolution_check=true" if strict else "an eval / inference load")

    # -- persistence -----------------------------------------------------------------------------
    def to_dict(self) -> dict[str, Any]:
        return encode(self)

    def _save_pretrained(self, save_directory: str | Path) -> None:
        """Writes ``config.json`` with the ``type`` discriminator, a concrete ``config_version`` (a saved ``null``
        would later be read as "no tag" = legacy) and the writing package's version; stripped fields are left out."""
        from .. import __version__
        d = self.to_dict()
        d["config_version"] = self.resolved_config_version()
        d["opentau_version"] = __version__ if __version__ != "unknown" else (self.opentau_version or __version__)
        strip_keys(d, REMOVED_POLICY_FIELDS)
        for k in DEPRECATED_LATENCY_FIELDS:          # still dataclass fields (old configs set them); never written
            d.pop(k, None)
        Path(save_directory).mkdir(parents=True, exist_ok=True)
        with open(Path(save_directory) / CONFIG_NAME, "w") as f:
            json.dump(d, f, indent=4)


    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "PreTrainedConfig":
        return decode(PreTrainedConfig if "type" in d else cls, d)

    @classmethod
    def from_pretrained(cls, pretrained_name_or_path: str | Path, *, cli_overrides: list[str] | None = None,
                        revision: str | None = None, **_unused) -> "PreTrainedConfig":
        """Loads a policy config from a directory, a file, or a ``repo@rev`` id in the local hub cache.

        Candidates in order: ``config.json``, then the whole-pipeline ``hf_config.json`` / ``train_config.json``, whose
        ``policy`` object is the policy config (published checkpoints historically carried ``hf_config.json`` alone).
        ``$ref`` includes are resolved once; deprecated and removed fields are reported with a ``DeprecationWarning``
        and dropped in memory -- the source file is never rewritten.  Reference:
        ``src/opentau/configs/policies.py:849-985``."""
        from ..utils.hub import resolve_local_or_hub, split_repo_revision
        from .codec import apply_overrides
        name = str(pretrained_name_or_path)
        if revision is not None and not os.path.exists(name) and "@" not in name:
            name = f"{name}@{revision}"
        root = resolve_local_or_hub(name)
        if root.is_file():
            config_file, nested = root, root.name != CONFIG_NAME and root.name in (HF_CONFIG_NAME, TRAIN_CONFIG_NAME)
        else:
            for filename in (CONFIG_NAME, HF_CONFIG_NAME, TRAIN_CONFIG_NAME):
                if (root / filename).is_file():
                    config_file, nested = root / filename, filename != CONFIG_NAME
                    break
            else:
                repo, rev = split_repo_revision(name)
                raise FileNotFoundError(f"None of {CONFIG_NAME}, {HF_CONFIG_NAME}, {TRAIN_CONFIG_NAME} found in "
                                        f"{root.resolve()}" + (f" (revision {rev!r} of {repo!r})" if rev else ""))
        raw = load_resolved_config_dict(config_file)
        if nested:
            raw = raw.get("policy")
            if not isinstance(raw, dict):
                raise FileNotFoundError(f"{config_file} carries no 'policy' object, so it cannot be read as a policy "
                                        f"config for {name}.")
        warn_deprecated_latency_fields_from_dict(raw, config_file)
        warn_removed_policy_fields_from_dict(raw, config_file)
        raw = dict(raw)
        strip_keys(raw, REMOVED_POLICY_FIELDS)
        if "config_version" not in raw:
            raw["config_version"] = None   # no tag: resolved against the weights when they are loaded
        if cli_overrides:
            raw = apply_overrides(raw, list(cli_overrides))
        return decode(PreTrainedConfig, raw)
