"""pi0.5 policy configuration (``type: pi05``), with the reference's field names and defaults
(OpenTau ``src/opentau/policies/pi05/configuration_pi05.py:97-234``).

B200-specific additions (all optional, absent from reference files): ``vlm`` / ``expert`` / ``vision``
geometry overrides for small test models, and ``discrete_action_vocab_size`` used when no FAST
processor is available offline.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ...configs.policies import PreTrainedConfig
from ...configs.types import FeatureType, NormalizationMode, PolicyFeature


@PreTrainedConfig.register_subclass("pi05")
@dataclass
class PI05Config(PreTrainedConfig):
    n_obs_steps: int = 1
    chunk_size: int = 50
    n_action_steps: int = 50
    normalization_mapping: dict[str, NormalizationMode] = field(default_factory=lambda: {
        "VISUAL": NormalizationMode.IDENTITY, "STATE": NormalizationMode.MIN_MAX,
        "ACTION": NormalizationMode.MEAN_STD})
    max_state_dim: int = 32
    max_action_dim: int = 32
    predict_response: bool = False
    state_type: str = "discrete"          # "discrete": 256-bin ids in the prompt | "continuous": state token
    resize_imgs_with_padding: tuple[int, int] = (224, 224)
    empty_cameras: int = 0
    prompt_max_length: int = 256
    response_indicator_max_length: int = 3
    discrete_action_indicator_max_length: int = 3
    response_max_length: int = 52
    discrete_action_max_length: int = 32
    discrete_action_tokenizer_path: str = "physical-intelligence/fast"
    discrete_action_vocab_size: int = 2048
    proj_width: int = 1024
    dropout: float = 0.1
    num_steps: int = 10
    max_delay: int = 0
    use_modality_embedding: bool = False
    attention_implementation: str = "eager"   # accepted for schema compatibility; one native kernel serves all
    freeze_vision_encoder: bool = True
    train_expert_only: bool = False
    train_vision_encoder_only: bool = False
    train_state_action_representation_only: bool = False
    knowledge_insulation: bool = True
    gradient_checkpointing: bool = False
    use_torch_compile: bool = True            # accepted and ignored: hot paths are hand-written kernels
    optimizer_lr: float = 2.5e-5
    optimizer_betas: tuple[float, float] = (0.9, 0.95)
    optimizer_eps: float = 1e-8
    optimizer_weight_decay: float = 1e-10
    scheduler_warmup_steps: int = 1000
    scheduler_decay_steps: int = 30000
    scheduler_decay_lr: float = 2.5e-6
    # {emitted action position: emitted state position} of a delta-joint-action mixture (post-index space): filled by
    # make_policy from the mixture's metadata, stored with the checkpoint, inverted in sample_actions.  JSON turns the
    # keys into strings; __post_init__ turns them back.
    delta_action_state_map: dict[int, int] | None = None
    # an openpi-style norm_stats.json that replaces the dataset-derived statistics of EVERY head (teacher replay)
    norm_stats_override_path: str | None = None
    tokenizer_path: str = "google/paligemma-3b-pt-224"
    # geometry overrides (dict of TowerConfig / SiglipConfig fields); None = the published sizes
    vlm: dict | None = None
    expert: dict | None = None
    vision: dict | None = None

    def __post_init__(self):
        super().__post_init__()
        if self.state_type not in ("discrete", "continuous"):
            raise ValueError(f"state_type must be 'discrete' or 'continuous', got {self.state_type!r}")
        if self.attention_implementation not in ("eager", "sdpa", "fa2", "flash_cuda", "tcgen05"):
            raise ValueError(f"unknown attention_implementation {self.attention_implementation!r}")
        if self.train_expert_only and not self.freeze_vision_encoder:
            raise ValueError("train_expert_only=True requires freeze_vision_encoder=True")
        if self.train_vision_encoder_only and (self.train_expert_only or self.freeze_vision_encoder):
            raise ValueError("train_vision_encoder_only is incompatible with train_expert_only / "
                             "freeze_vision_encoder")
        if self.train_state_action_representation_only and (self.train_expert_only or self.train_vision_encoder_only):
            raise ValueError("train_state_action_representation_only is mutually exclusive with "
                             "train_expert_only and train_vision_encoder_only")
        if self.delta_action_state_map is not None:
            try:
                self.delta_action_state_map = {int(a): int(b) for a, b in self.delta_action_state_map.items()}
            except (TypeError, ValueError, AttributeError) as exc:
                raise ValueError("`delta_action_state_map` must map int action positions to int state positions, got "
                                 f"{self.delta_action_state_map!r}") from exc
            if any(a < 0 or b < 0 for a, b in self.delta_action_state_map.items()):
                raise ValueError(f"`delta_action_state_map` positions must be non-negative, got {self.delta_action_state_map!r}")
        self.validate_action_horizon()

    def validate_features(self) -> None:
        for i in range(self.empty_cameras):
            self.input_features[f"empty_camera{i}"] = PolicyFeature(
                FeatureType.VISUAL, (3, *self.resize_imgs_with_padding))


@PreTrainedConfig.register_subclass("pi05_continuous_state")
@dataclass
class PI05ContinuousStateConfig(PI05Config):
    state_type: str = "continuous"
