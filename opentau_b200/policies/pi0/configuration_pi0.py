"""pi0 configuration (``type: pi0``): PaliGemma + Gemma-300M expert with plain RMSNorm, a state token and an
action||time MLP in the suffix, optional advantage-conditioned prompts (RECAP) and advantage-weighted
regression (reference ``src/opentau/policies/pi0/configuration_pi0.py``)."""

from __future__ import annotations

from dataclasses import dataclass

from ...configs.policies import PreTrainedConfig
from ..pi05.configuration_pi05 import PI05Config


@PreTrainedConfig.register_subclass("pi0")
@dataclass
class PI0Config(PI05Config):
    state_type: str = "continuous"
    knowledge_insulation: bool = False
    tokenizer_max_length: int = 48
    prompt_max_length: int = 48
    advantage: str = "use"               # "ignore" | "on" | "use"
    advantage_threshold: float = 0.0
    use_awr: bool = False
    awr_max_weight: float = 10.0
    use_torch_compile: bool = False

    _deprecated_fields = ("job_name",)

    def __post_init__(self):
        super().__post_init__()
        if self.advantage not in ("ignore", "on", "use"):
            raise ValueError(f"advantage must be 'ignore', 'on' or 'use', got {self.advantage!r}")
        if self.attention_implementation == "flash_cuda":
            raise ValueError("pi0 does not offer the flash_cuda attention option")
        self.prompt_max_length = self.tokenizer_max_length
