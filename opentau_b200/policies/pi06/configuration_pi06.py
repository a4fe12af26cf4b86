"""pi0.6 configuration (``type: pi06``): Gemma-3-4B backbone, 448x448 images pooled to 256 tokens per
camera, ~860 M action expert (width 1280), 5 flow-matching steps, discrete state only
(reference ``src/opentau/policies/pi06/configuration_pi06.py:38-276``)."""

from __future__ import annotations

from dataclasses import dataclass, field

from ...configs.policies import PreTrainedConfig
from ...configs.types import NormalizationMode
from ..pi05.configuration_pi05 import PI05Config


@PreTrainedConfig.register_subclass("pi06")
@dataclass
class PI06Config(PI05Config):
    resize_imgs_with_padding: tuple[int, int] = (448, 448)
    proj_width: int = 1280
    num_steps: int = 5
    state_type: str = "discrete"
    use_modality_embedding: bool = False
    tokenizer_path: str = "google/gemma-3-4b-pt"
    use_torch_compile: bool = False
    vlm_config: dict | None = None      # nested wrapper overrides: {"text": {...}, "expert": {...}, "vision": {...}}

    def __post_init__(self):
        super().__post_init__()
        if self.state_type != "discrete":
            raise ValueError("pi06 supports the discrete state representation only")
        if self.use_modality_embedding:
            raise ValueError("pi06 has no modality embedding")
