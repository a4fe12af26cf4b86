"""cosmos3_nano: the same policy over the 8B Qwen3-VL backbone (36 layers); defaults only
(reference ``src/opentau/policies/cosmos3_nano``)."""

from __future__ import annotations

from dataclasses import dataclass

from ...configs.policies import PreTrainedConfig
from ..cosmos3.configuration_cosmos3 import Cosmos3Config


@PreTrainedConfig.register_subclass("cosmos3_nano")
@dataclass
class Cosmos3NanoConfig(Cosmos3Config):
    pretrained_backbone_repo_id: str = "TensorAuto/cosmos3-reason-8b"
    expert_num_hidden_layers: int = 36
    tokenizer_path: str = "Qwen/Qwen3-VL-8B-Instruct"

    def __post_init__(self):
        if self.backbone is None:
            self.backbone = dict(hidden_size=4096, num_hidden_layers=36, num_attention_heads=32,
                                 num_key_value_heads=8, head_dim=128, intermediate_size=12288)
        super().__post_init__()
