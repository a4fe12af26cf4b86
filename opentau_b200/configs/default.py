"""Dataset, mixture, logging and evaluation configuration blocks.

Field names and defaults follow the reference schema (OpenTau ``src/opentau/configs/default.py:53-1011``)
so existing JSON configs parse; B200-specific additions are grouped in :class:`DistributedConfig`.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass
class ImageTransformConfig:
    weight: float = 1.0
    type: str = "Identity"
    kwargs: dict[str, Any] = field(default_factory=dict)


@dataclass
class ImageTransformsConfig:
    enable: bool = False
    max_num_transforms: int = 3
    random_order: bool = False
    tfs: dict[str, ImageTransformConfig] = field(default_factory=lambda: {
        "brightness": ImageTransformConfig(1.0, "ColorJitter", {"brightness": (0.8, 1.2)}),
        "contrast": ImageTransformConfig(1.0, "ColorJitter", {"contrast": (0.8, 1.2)}),
        "saturation": ImageTransformConfig(1.0, "ColorJitter", {"saturation": (0.5, 1.5)}),
        "hue": ImageTransformConfig(1.0, "ColorJitter", {"hue": (-0.05, 0.05)}),
        "sharpness": ImageTransformConfig(1.0, "SharpnessJitter", {"sharpness": (0.5, 1.5)}),
    })


@dataclass
class DatasetConfig:
    """One entry of the mixture: a LeRobot dataset (``repo_id``), a VQA set (``vqa``) or, new here, a
    ``synthetic`` generator spec used for benchmarks and tests."""

    repo_id: str | None = None
    vqa: str | None = None
    synthetic: dict[str, Any] | None = None
    root: str | None = None
    episodes: list[int] | None = None
    excluded_episodes: list[int] | None = None
    image_transforms: ImageTransformsConfig = field(default_factory=ImageTransformsConfig)
    revision: str | None = None
    use_imagenet_stats: bool = True
    video_backend: str = "pyav"
    stats: dict[str, dict[str, list]] | None = None
    data_features_name_mapping: dict[str, str] | None = None
    prompt_substitutions: dict[str, list[str]] | None = None
    robot_type: str | None = None
    control_mode: str | None = None
    tolerance_s: float | None = None
    skip_timestamp_check: bool | None = None
    val_split_ratio: float | None = None
    state_index: list[int] | None = None
    action_index: list[int] | None = None
    use_delta_joint_actions: bool = False
    delta_action_state_map: dict[str, int] | None = None

    def __post_init__(self):
        n = sum(x is not None for x in (self.repo_id, self.vqa, self.synthetic))
        if n != 1:
            raise ValueError("exactly one of `repo_id`, `vqa` or `synthetic` must be set")
        if self.tolerance_s is not None and self.tolerance_s < 0:
            raise ValueError("tolerance_s must be >= 0")
        if self.val_split_ratio is not None and not (0.0 <= self.val_split_ratio < 1.0):
            raise ValueError("val_split_ratio must be in [0, 1)")
        if self.prompt_substitutions is not None:
            if self.repo_id is None:
                raise ValueError("prompt_substitutions is only available for LeRobot datasets")
            for k, v in self.prompt_substitutions.items():
                if not isinstance(k, str) or k == "$ref":
                    raise ValueError(f"bad prompt_substitutions key {k!r}")
                if not v or any((not isinstance(s, str)) or not s for s in v):
                    raise ValueError(f"prompt_substitutions[{k!r}] must be a non-empty list of non-empty strings")
        if self.use_delta_joint_actions and not self.delta_action_state_map:
            raise ValueError("use_delta_joint_actions requires delta_action_state_map")
        for name in ("state_index", "action_index"):
            idx = getattr(self, name)
            if idx is not None and (len(set(idx)) != len(idx) or any(i < 0 for i in idx)):
                raise ValueError(f"{name} must hold unique non-negative indices")

    @property
    def name(self) -> str:
        return self.repo_id or self.vqa or f"synthetic:{(self.synthetic or {}).get('name', 'default')}"


@dataclass
class DatasetMixtureConfig:
    datasets: list[DatasetConfig] = field(default_factory=list)
    weights: list[float] | None = None
    #: Hz at which every dataset's actions are resampled; None = each dataset at its own fps
    action_freq: float | None = None
    image_resample_strategy: str = "nearest"
    vector_resample_strategy: str = "nearest"
    val_split_ratio: float = 0.05
    n_obs_history: int | None = None
    history_state_drop_prob: float = 0.3
    subgoal_drop_prob: float = 0.75
    subgoal_end_of_segment_prob: float = 0.25
    response_drop_prob: float = 0.3
    metadata_drop_all_prob: float = 0.15
    metadata_drop_each_prob: float = 0.05
    val_enable_optional_key_dropout: bool = False
    val_enable_prompt_substitution: bool = False
    require_non_empty_robot_type: bool = False
    require_non_empty_control_mode: bool = False
    emit_fps: bool = False
    tolerance_s: float = 1e-4
    skip_timestamp_check: bool = False
    delta_stats_max_rows: int | None = None

    def __post_init__(self):
        if self.weights is not None and len(self.weights) != len(self.datasets):
            raise ValueError("`weights` must have one entry per dataset")
        if self.weights is not None and any(w < 0 for w in self.weights):
            raise ValueError("mixture weights must be non-negative")
        if self.image_resample_strategy not in ("nearest", "linear"):
            raise ValueError("image_resample_strategy must be 'nearest' or 'linear'")
        if self.vector_resample_strategy not in ("nearest", "linear"):
            raise ValueError("vector_resample_strategy must be 'nearest' or 'linear'")
        if not (0.0 <= self.val_split_ratio < 1.0):
            raise ValueError("val_split_ratio must be in [0, 1)")
        if self.action_freq is not None and not self.action_freq > 0:
            raise ValueError(f"action_freq must be positive or None, got {self.action_freq}")
        for p in ("history_state_drop_prob", "subgoal_drop_prob", "subgoal_end_of_segment_prob",
                  "response_drop_prob", "metadata_drop_all_prob", "metadata_drop_each_prob"):
            if not (0.0 <= getattr(self, p) <= 1.0):
                raise ValueError(f"{p} must be a probability")


@dataclass
class WandBConfig:
    enable: bool = False
    entity: str | None = None
    project: str = "opentau"
    run_id: str | None = None
    name: str | None = None
    notes: str | None = None
    tags: list[str] = field(default_factory=list)
    group: str | None = None
    job_type: str | None = None
    mode: str | None = None            # online | offline | disabled
    allow_resume: bool = True
    disable_artifact: bool = False


@dataclass
class EvalConfig:
    n_episodes: int = 16
    batch_size: int = 16
    use_async_envs: bool = True
    max_episodes_rendered: int = 16
    grid_size: tuple[int, int] | None = None
    video_fps: int | None = None
    video_crf: int = 23
    recording_root: str | None = None
    seed: int | None = None
    decorrelate_rank_seeds: bool = True
    goal_frames_dir: str | None = None
    seed_list: list[int] | None = None
    dataset_repo_id: str | None = None
    robot_type: str | None = None
    control_mode: str | None = None

    def __post_init__(self):
        if self.batch_size > self.n_episodes:
            raise ValueError(f"eval.batch_size ({self.batch_size}) must be <= eval.n_episodes ({self.n_episodes})")
        if self.seed_list is not None and len(self.seed_list) < self.n_episodes:
            raise ValueError("seed_list must provide one seed per episode")


@dataclass
class DistributedConfig:
    """B200 data/tensor/context-parallel layout (replaces the reference's accelerate YAML surface).

    ``strategy``: ``ddp`` (replicated optimizer) | ``zero2`` / ``fsdp`` (sharded optimizer state);
    ``comm``: ``p2p`` (fused peer-memory kernels) | ``nccl`` (library collectives) | ``auto``;
    ``tp`` / ``cp``: tensor- and context-parallel degrees (product with the data-parallel degree = world).
    """

    strategy: str = "zero2"
    comm: str = "auto"
    tp: int = 1
    cp: int = 1
    gradient_clipping: float | None = None

    def __post_init__(self):
        if self.strategy not in ("ddp", "zero1", "zero2", "zero3", "fsdp", "deepspeed"):
            raise ValueError(f"unknown distributed strategy {self.strategy!r}")
        if self.comm not in ("auto", "p2p", "nccl"):
            raise ValueError(f"unknown comm backend {self.comm!r}")

    @classmethod
    def from_accelerate_yaml(cls, path: str) -> "DistributedConfig":
        """Maps an ``accelerate`` config file (``distributed_type`` MULTI_GPU / DEEPSPEED / FSDP) onto this
        block, so ``opentau-train --accelerate-config X`` keeps working."""
        import yaml
        with open(path) as f:
            y = yaml.safe_load(f) or {}
        dt = str(y.get("distributed_type", "MULTI_GPU")).upper()
        clip = None
        if dt == "DEEPSPEED":
            ds = y.get("deepspeed_config", {}) or {}
            stage = int(ds.get("zero_stage", 2))
            strategy = {0: "ddp", 1: "zero1", 2: "zero2", 3: "zero3"}.get(stage, "zero2")
            clip = ds.get("gradient_clipping")
        elif dt == "FSDP":
            strategy = "fsdp"
        else:
            strategy = "ddp"
        return cls(strategy=strategy, gradient_clipping=float(clip) if clip is not None else None)
