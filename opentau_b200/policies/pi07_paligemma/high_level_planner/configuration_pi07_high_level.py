"""``type: pi07_paligemma_high_level_planner`` (reference
``src/opentau/policies/pi07_paligemma/high_level_planner/configuration_pi07_high_level.py:34-200``)."""

from __future__ import annotations

from dataclasses import dataclass

from ....configs.policies import PreTrainedConfig
from ...pi07.high_level_planner.configuration_pi07_high_level import PI07HighLevelPlannerConfig


@PreTrainedConfig.register_subclass("pi07_paligemma_high_level_planner")
@dataclass
class PI07PaligemmaHighLevelPlannerConfig(PI07HighLevelPlannerConfig):
    resize_imgs_with_padding: tuple[int, int] = (224, 224)
    tokenizer_path: str = "google/paligemma-3b-pt-224"
    # fields the PaliGemma wrapper reads
    expert: dict | None = None
    discrete_action_vocab_size: int = 8
    train_expert_only: bool = False
    train_vision_encoder_only: bool = False
    train_state_action_representation_only: bool = False
    disable_action_expert: bool = True
