"""pi0.7 high-level planner on PaliGemma (reference
``src/opentau/policies/pi07_paligemma/high_level_planner/modeling_pi07_high_level.py``): memory + subtask text
generation with the PaliGemma backbone, no action expert."""

from __future__ import annotations

from ...pi05.modeling_pi05 import PaliGemmaWithExpertModel, gemma_2b_config
from ...pi07.high_level_planner.modeling_pi07_high_level import PI07HighLevelPlannerModel, PI07HighLevelPlannerPolicy
from .configuration_pi07_high_level import PI07PaligemmaHighLevelPlannerConfig


class PI07PaligemmaHighLevelPlannerModel(PI07HighLevelPlannerModel):
    wrapper_attr = "paligemma_with_expert"

    def build_wrapper(self, config):
        return PaliGemmaWithExpertModel(config)


class PI07PaligemmaHighLevelPlannerPolicy(PI07HighLevelPlannerPolicy):
    config_class = PI07PaligemmaHighLevelPlannerConfig
    name = "pi07_paligemma_high_level_planner"
    model_class = PI07PaligemmaHighLevelPlannerModel

    @staticmethod
    def _vocab_size(config) -> int:
        return gemma_2b_config(**(config.vlm or {})).vocab_size
