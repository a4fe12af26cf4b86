"""pi0.7 low-level controller configuration (``type: pi07_low_level``)
(reference ``src/opentau/policies/pi07/low_level/configuration_pi07_low_level.py:144-283``)."""

from __future__ import annotations

from dataclasses import dataclass

from ....configs.policies import PreTrainedConfig
from ...pi06.configuration_pi06 import PI06Config


@PreTrainedConfig.register_subclass("pi07_low_level")
@dataclass
class PI07LowLevelConfig(PI06Config):
    n_obs_steps: int = 6
    history_interval: int = 1
    prompt_max_length: int = 256
    discrete_action_max_length: int = 32
    metadata_max_length: int = 52
    response_max_length: int = 52
    proj_width: int = 1280
    per_group_projection: bool = False
    num_steps: int = 5
    spacetime_layer_stride: int = 4
    use_torch_compile: bool = True
    warn_outlier_threshold: float = 32.0
    num_subgoal_cameras: int = 0
    keep_history_tokens: bool = False      # keep every frame's tokens in the decoder (long-context variant)

    def __post_init__(self):
        super().__post_init__()
        if self.n_obs_steps < 1:
            raise ValueError("n_obs_steps must be >= 1")
        if self.history_interval < 1:
            raise ValueError("history_interval must be >= 1")

    @property
    def observation_delta_indices(self):
        return [-(self.n_obs_steps - 1 - i) * self.history_interval for i in range(self.n_obs_steps)]
