"""cosmos3 configuration (``type: cosmos3``): frozen Qwen3-VL backbone + trainable Qwen3 action expert
(reference ``src/opentau/policies/cosmos3/configuration_cosmos3.py:48-301``).  ``backbone`` / ``vision`` are
B200-side geometry overrides (the reference reads the geometry from the pretrained HF config)."""

from __future__ import annotations

from dataclasses import dataclass, field

from ...configs.policies import PreTrainedConfig
from ...configs.types import NormalizationMode


@PreTrainedConfig.register_subclass("cosmos3")
@dataclass
class Cosmos3Config(PreTrainedConfig):
    n_obs_steps: int = 1
    chunk_size: int = 50
    n_action_steps: int = 50
    normalization_mapping: dict[str, NormalizationMode] = field(default_factory=lambda: {
        "VISUAL": NormalizationMode.IDENTITY, "STATE": NormalizationMode.MEAN_STD,
        "ACTION": NormalizationMode.MEAN_STD})
    max_state_dim: int = 32
    max_action_dim: int = 32
    proj_width: int = 1024
    prompt_max_length: int = 256
    empty_cameras: int = 0
    num_steps: int = 10
    max_delay: int = 0
    pretrained_backbone_repo_id: str = "TensorAuto/cosmos3-reason-32b"
    load_pretrained_backbone: bool = True
    image_resize: int = 224
    attention_implementation: str = "sdpa"
    freeze_vision_encoder: bool = True
    train_expert_only: bool = True
    train_vision_encoder_only: bool = False
    train_state_action_representation_only: bool = False
    gradient_checkpointing: bool = False
    dropout: float = 0.1
    condition_on_layer: int | None = None
    expert_hidden_size: int = 1024
    expert_intermediate_size: int = 2048
    expert_num_hidden_layers: int = 64
    expert_num_attention_heads: int = 16
    expert_num_key_value_heads: int = 8
    expert_head_dim: int = 128
    expert_adarms_cond_dim: int = 256
    expert_rms_norm_eps: float = 1e-6
    expert_rope_theta: float = 5e6
    optimizer_lr: float = 2.5e-5
    optimizer_betas: tuple[float, float] = (0.9, 0.95)
    optimizer_eps: float = 1e-8
    optimizer_weight_decay: float = 1e-10
    scheduler_warmup_steps: int = 1000
    scheduler_decay_steps: int = 30000
    scheduler_decay_lr: float = 2.5e-6
    use_torch_compile: bool = False
    tokenizer_path: str = "Qwen/Qwen3-VL-32B-Instruct"
    backbone: dict | None = None
    vision: dict | None = None
    tensor_parallel: int = 1

    def __post_init__(self):
        super().__post_init__()
        if self.attention_implementation in ("flash_cuda", "fa2"):
            raise ValueError("cosmos3 accepts attention_implementation 'eager' or 'sdpa'")
        if self.train_vision_encoder_only and (self.train_expert_only or self.freeze_vision_encoder):
            raise ValueError("train_vision_encoder_only conflicts with train_expert_only / freeze_vision_encoder")
        self.validate_action_horizon()

    @property
    def resize_imgs_with_padding(self) -> tuple[int, int]:
        return (self.image_resize, self.image_resize)
