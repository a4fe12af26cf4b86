"""``type: pi07_paligemma_low_level`` (reference
``src/opentau/policies/pi07_paligemma/low_level/configuration_pi07_low_level.py:36-260``): the pi0.7 low-level
controller with PaliGemma geometry — 224x224 images, Gemma-2B backbone, 300 M expert of width 1024, 10 steps."""

from __future__ import annotations

from dataclasses import dataclass

from ....configs.policies import PreTrainedConfig
from ...pi07.low_level.configuration_pi07_low_level import PI07LowLevelConfig


@PreTrainedConfig.register_subclass("pi07_paligemma_low_level")
@dataclass
class PI07PaligemmaLowLevelConfig(PI07LowLevelConfig):
    resize_imgs_with_padding: tuple[int, int] = (224, 224)
    proj_width: int = 1024
    num_steps: int = 10
    tokenizer_path: str = "google/paligemma-3b-pt-224"
