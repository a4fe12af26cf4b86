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

from ..constants import CONFIG_NAME
from .codec import ChoiceRegistry, decode, encode
from .types import FeatureType, NormalizationMode, PolicyFeature

CURRENT_CONFIG_VERSION = 1
OPENPI_EPS = 1e-6   # normalization epsilon for config_version >= 1
LEGACY_EPS = 1e-8   # epsilon for checkpoints without a version


@dataclass
class PreTrainedConfig(ChoiceRegistry, abc.ABC):
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

    @property
    def zero_range_centers_on_zero(self) -> bool:
        """New-format checkpoints map a zero-range dim to 0; legacy ones to -1."""
        return (self.config_version or 0) >= 1

    @property
    def normalization_epsilon(self) -> float:
        return OPENPI_EPS if (self.config_version or 0) >= 1 else LEGACY_EPS

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
        from .. import __version__
        d = self.to_dict()
        if d.get("config_version") is None:
            d["config_version"] = CURRENT_CONFIG_VERSION
        d["opentau_version"] = __version__
        Path(save_directory).mkdir(parents=True, exist_ok=True)
        with open(Path(save_directory) / CONFIG_NAME, "w") as f:
            json.dump(d, f, indent=4)

    save_pretrained = _save_pretrained

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "PreTrainedConfig":
        return decode(PreTrainedConfig if "type" in d else cls, d)

    @classmethod
    def from_pretrained(cls, pretrained_name_or_path: str | Path, *, cli_overrides: list[str] | None = None,
                        **_unused) -> "PreTrainedConfig":
        """Loads ``config.json`` from a local directory (``repo@rev`` hub ids need network and raise)."""
        from .codec import apply_overrides
        from ..utils.hub import resolve_local_or_hub
        path = resolve_local_or_hub(str(pretrained_name_or_path), CONFIG_NAME)
        with open(path) as f:
            raw = json.load(f)
        if "config_version" not in raw:
            raw["config_version"] = None  # legacy provenance: keep eps 1e-8 / centre -1 behaviour
        if cli_overrides:
            raw = apply_overrides(raw, list(cli_overrides))
        return decode(PreTrainedConfig, raw)
