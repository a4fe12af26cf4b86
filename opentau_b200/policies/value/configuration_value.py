"""Value-model configuration (``type: value``; reference ``src/opentau/policies/value/configuration_value.py:36-171``).

``vlm`` / ``vision`` are geometry overrides for small test models; None = Gemma-3 270M and SigLIP2-so400m.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ...configs.policies import PreTrainedConfig
from ...configs.reward import RewardConfig
from ...configs.types import FeatureType, NormalizationMode, PolicyFeature


@PreTrainedConfig.register_subclass("value")
@dataclass
class ValueConfig(PreTrainedConfig):
    n_obs_steps: int = 1
    chunk_size: int = 50
    normalization_mapping: dict[str, NormalizationMode] = field(default_factory=lambda: {
        "VISUAL": NormalizationMode.IDENTITY, "STATE": NormalizationMode.MIN_MAX,
        "ACTION": NormalizationMode.MEAN_STD})
    max_state_dim: int = 32
    resize_imgs_with_padding: tuple[int, int] = (224, 224)
    empty_cameras: int = 0
    prompt_max_length: int = 48
    response_max_length: int = 52
    reward_config: RewardConfig = field(default_factory=RewardConfig)
    optimizer_lr: float = 2.5e-5
    optimizer_betas: tuple[float, float] = (0.9, 0.95)
    optimizer_eps: float = 1e-8
    optimizer_weight_decay: float = 1e-10
    scheduler_warmup_steps: int = 1_000
    scheduler_decay_steps: int = 30_000
    scheduler_decay_lr: float = 2.5e-6
    tokenizer_path: str = "google/gemma-3-270m"
    vlm: dict | None = None
    vision: dict | None = None

    action_horizon_delay_field = None

    def __post_init__(self):
        super().__post_init__()
        if self.n_obs_steps != 1:
            raise ValueError(f"Multiple observation steps not handled yet. Got `nobs_steps={self.n_obs_steps}`")
        rc = self.reward_config
        if not rc.reward_normalizer + rc.C_neg < abs(rc.C_neg):
            raise ValueError("max episode length must stay below |C_neg| so failed and successful episodes "
                             "occupy disjoint return ranges")

    def validate_features(self) -> None:
        for i in range(self.empty_cameras):
            self.input_features[f"observation.images.empty_camera_{i}"] = PolicyFeature(
                FeatureType.VISUAL, (3, 480, 640))
