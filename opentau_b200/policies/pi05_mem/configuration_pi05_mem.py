"""pi0.5-MEM configuration (``type: pi05_mem``; reference ``src/opentau/policies/pi05_mem/configuration_pi05.py:38-392``):
pi0.5 with a video history per camera (space-time SigLIP, or per-frame SigLIP + STSS motion module), one continuous
state token per history step, and interleaved multimodal RoPE on the video patches."""

from __future__ import annotations

from dataclasses import dataclass

from ...configs.policies import PreTrainedConfig
from ..pi05.configuration_pi05 import PI05Config


@PreTrainedConfig.register_subclass("pi05_mem")
@dataclass
class PI05MemConfig(PI05Config):
    n_obs_steps: int = 8
    history_interval: int = 1                 # environment steps between two history frames
    state_type: str = "continuous"            # one projected token per history step
    rope_type: str = "mrope_interleaved"      # "rope": scalar positions (checkpoints trained before MRoPE)
    spacetime_layer_stride: int = 4
    use_motion: bool = False                  # per-frame SigLIP + STSS motion residual instead of space-time attention
    motion_insert_layer: int | None = None
    motion_hidden_dim: int = 256
    motion_window: tuple[int, int, int] = (5, 9, 9)
    motion_corr_func: str = "cosine"
    motion_n_encoders: int = 1
    motion_norm: str = "groupnorm"
    motion_int_mode: str = "lite"
    motion_zero_init: bool = True
    use_torch_compile: bool = False

    def __post_init__(self):
        super().__post_init__()
        if self.rope_type not in ("rope", "mrope_interleaved"):
            raise ValueError(f"`rope_type` must be one of 'rope'/'mrope_interleaved', got {self.rope_type!r}.")
        if self.n_obs_steps < 1 or self.history_interval < 1:
            raise ValueError("n_obs_steps and history_interval must be >= 1")
        if self.predict_response:
            raise ValueError("pi05_mem has no response head")
        if self.motion_corr_func not in ("cosine", "dotproduct", "dotproduct_softmax"):
            raise ValueError(f"unknown motion_corr_func {self.motion_corr_func!r}")

    @property
    def observation_delta_indices(self) -> list[int]:
        return [-(self.n_obs_steps - 1 - i) * self.history_interval for i in range(self.n_obs_steps)]
