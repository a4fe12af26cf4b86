"""pi0.7 high-level planner configuration (``type: pi07_high_level``): Gemma-3 backbone without an action
expert, trained with CE over memory + subtask text
(reference ``src/opentau/policies/pi07/high_level_planner/configuration_pi07_high_level.py:112-194``)."""

from __future__ import annotations

from dataclasses import dataclass, field

from ....configs.policies import PreTrainedConfig
from ....configs.types import NormalizationMode


@PreTrainedConfig.register_subclass("pi07_high_level")
@dataclass
class PI07HighLevelPlannerConfig(PreTrainedConfig):
    n_obs_steps: int = 1
    normalization_mapping: dict[str, NormalizationMode] = field(default_factory=lambda: {
        "VISUAL": NormalizationMode.IDENTITY, "STATE": NormalizationMode.MIN_MAX,
        "ACTION": NormalizationMode.MEAN_STD})
    max_state_dim: int = 32
    resize_imgs_with_padding: tuple[int, int] = (448, 448)
    empty_cameras: int = 0
    prompt_max_length: int = 256
    memory_max_length: int = 52
    response_max_length: int = 52
    metadata_max_length: int = 52
    subtask_indicator_max_length: int = 4
    memory_indicator_max_length: int = 4
    discrete_action_tokenizer_path: str = "physical-intelligence/fast"
    dropout: float = 0.1
    attention_implementation: str = "eager"
    freeze_vision_encoder: bool = True
    gradient_checkpointing: bool = False
    vlm_config: dict | None = None
    vlm: dict | None = None
    vision: dict | None = None
    optimizer_lr: float = 2.5e-5
    optimizer_betas: tuple[float, float] = (0.9, 0.95)
    optimizer_eps: float = 1e-8
    optimizer_weight_decay: float = 1e-10
    scheduler_warmup_steps: int = 1000
    scheduler_decay_steps: int = 30000
    scheduler_decay_lr: float = 2.5e-6
    tokenizer_path: str = "google/gemma-3-4b-pt"
    action_horizon_delay_field = None

    def __post_init__(self):
        super().__post_init__()
        if self.attention_implementation not in ("eager", "sdpa", "fa2", "tcgen05"):
            raise ValueError(f"unsupported attention_implementation {self.attention_implementation!r}")
