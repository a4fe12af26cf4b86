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
    delta_action_state_map: dict[Any, int] | None = None      # {action dim: state dim}, parquet index space

    def __post_init__(self):
        n = sum(x is not None for x in (self.repo_id, self.vqa, self.synthetic))
        if n != 1:
            raise ValueError("exactly one of `repo_id`, `vqa` or `synthetic` must be set")
        who = self.name
        self._validate_index_and_delta()
        if self.tolerance_s is not None and self.tolerance_s < 0:
            raise ValueError(f"`DatasetConfig.tolerance_s` must be >= 0 (or None to inherit), got {self.tolerance_s} "
                             f"for {who}.")
        if self.val_split_ratio is not None and not (0.0 <= self.val_split_ratio <= 1.0):
            raise ValueError(f"`DatasetConfig.val_split_ratio` must be in [0, 1] (or None to inherit), got "
                             f"{self.val_split_ratio} for {who}.")
        if self.prompt_substitutions is not None:
            if self.repo_id is None:
                raise ValueError(f"`DatasetConfig.prompt_substitutions` only applies to LeRobot datasets (`repo_id`); "
                                 f"{who!r} builds its own prompt.")
            for task, subs in self.prompt_substitutions.items():
                if not isinstance(task, str):
                    raise ValueError(f"`prompt_substitutions` keys must be on-disk task strings, got {task!r} for {who}.")
                if task == "$ref":
                    raise ValueError("`prompt_substitutions` cannot map a task literally named '$ref': the config "
                                     "loader treats any JSON object containing a '$ref' key as a file include.")
                if not isinstance(subs, list) or len(subs) == 0:
                    raise ValueError(f"`prompt_substitutions[{task!r}]` must be a non-empty list of strings, got "
                                     f"{subs!r} for {who}.")
                if not all(isinstance(x, str) and x for x in subs):
                    raise ValueError(f"`prompt_substitutions[{task!r}]` contains empty or non-string entries: {subs!r} "
                                     f"for {who}. A matching sample's task is ALWAYS replaced, so an empty substitute "
                                     "would silently train on an empty prompt.")

    def _validate_index_and_delta(self) -> None:
        """``state_index`` / ``action_index`` / delta-action fields.  The keys and values of ``delta_action_state_map``
        are coerced to ``int``: a JSON config round-trips object keys as strings (``{"0": 0}``), and a string key would
        silently match no action dim, leaving every dim absolute."""
        who = self.name
        lerobot = self.repo_id is not None
        for name in ("state_index", "action_index"):
            index = getattr(self, name)
            if index is None:
                continue
            if not lerobot:
                raise ValueError(f"`DatasetConfig.{name}` only applies to LeRobot datasets (`repo_id`); {who!r} emits "
                                 "pre-shaped tensors.")
            if not isinstance(index, list) or not index:
                raise ValueError(f"`DatasetConfig.{name}` must be a non-empty list of column indices (or None to keep "
                                 f"every dim), got {index!r} for {who}.")
            if not all(isinstance(i, int) and not isinstance(i, bool) and i >= 0 for i in index):
                raise ValueError(f"`DatasetConfig.{name}` entries must be non-negative ints, got {index!r} for {who}.")
            if len(set(index)) != len(index):
                dupes = sorted({i for i in index if index.count(i) > 1})
                raise ValueError(f"`DatasetConfig.{name}` contains duplicate indices {dupes} for {who}. Repeating a "
                                 "column is almost always a typo; list each index once.")
        if self.delta_action_state_map is not None:
            if not lerobot:
                raise ValueError(f"`DatasetConfig.delta_action_state_map` only applies to LeRobot datasets (`repo_id`); "
                                 f"{who!r} has no proprioceptive state.")
            try:
                coerced = {int(a): int(v) for a, v in self.delta_action_state_map.items()}
            except (TypeError, ValueError) as exc:
                raise ValueError("`DatasetConfig.delta_action_state_map` must map int action dims to int state dims, "
                                 f"got {self.delta_action_state_map!r} for {who}.") from exc
            if any(a < 0 or v < 0 for a, v in coerced.items()):
                raise ValueError("`DatasetConfig.delta_action_state_map` indices must be non-negative, got "
                                 f"{self.delta_action_state_map!r} for {who}.")
            self.delta_action_state_map = coerced
        if self.use_delta_joint_actions and not self.delta_action_state_map:
            raise ValueError("`DatasetConfig.use_delta_joint_actions=True` requires a non-empty "
                             f"`delta_action_state_map` (at least one action dim), but none was given for {who}.")
        if self.delta_action_state_map and not self.use_delta_joint_actions:
            raise ValueError(f"`DatasetConfig.delta_action_state_map` is set but `use_delta_joint_actions` is False for "
                             f"{who}, so the mapping would be silently ignored and actions would train as absolute. "
                             "Set the flag, or remove the mapping.")

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
        if not (0.0 <= self.val_split_ratio <= 1.0):
            raise ValueError(f"`val_split_ratio` must be between 0 and 1, got {self.val_split_ratio}.")
        if self.action_freq is not None and not self.action_freq > 0:
            raise ValueError(f"action_freq must be positive or None, got {self.action_freq}")
        if self.tolerance_s < 0:
            raise ValueError(f"`tolerance_s` must be >= 0, got {self.tolerance_s}.")
        if self.n_obs_history is not None and (not isinstance(self.n_obs_history, int) or self.n_obs_history < 1):
            raise ValueError(f"`n_obs_history` must be None or a positive integer, got {self.n_obs_history}.")
        m = self.delta_stats_max_rows
        if m is not None and (not isinstance(m, int) or isinstance(m, bool) or m < 1):
            raise ValueError(f"`delta_stats_max_rows` must be None (uncapped) or a positive integer, got {m!r}.")
        for p in ("history_state_drop_prob", "subgoal_drop_prob", "subgoal_end_of_segment_prob",
                  "response_drop_prob", "metadata_drop_all_prob", "metadata_drop_each_prob"):
            if not (0.0 <= getattr(self, p) <= 1.0):
                raise ValueError(f"{p} must be a probability")


@dataclass
class WandBConfig:
    """Weights & Biases logging.  ``on_resume``: what happens when a run that has a ``run_id`` resumes from a checkpoint
    step: ``"fork"`` (default) starts a NEW run branching from the parent at that step (``fork_from``; the parent stays
    immutable, a job requeued N times leaves a chain of N linked runs), ``"continue"`` resumes the same run in place.
    ``allow_resume`` is the deprecated spelling (True -> continue, False -> fork)."""

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
    on_resume: str = "fork"
    allow_resume: bool | None = None
    disable_artifact: bool = False
    disable_video: bool = False

    def __post_init__(self):
        import warnings
        if self.allow_resume is not None:
            warnings.warn("`wandb.allow_resume` is deprecated; use `wandb.on_resume='fork'|'continue'`.", FutureWarning,
                          stacklevel=2)
            mapped = "continue" if self.allow_resume else "fork"
            if self.on_resume == "fork":
                self.on_resume = mapped
            elif self.on_resume != mapped:
                warnings.warn(f"Both `allow_resume`={self.allow_resume} and `on_resume`='{self.on_resume}' are set; "
                              "using `on_resume`.", FutureWarning, stacklevel=2)
            self.allow_resume = None
        if self.on_resume not in ("fork", "continue"):
            raise ValueError(f"`on_resume` must be 'fork' or 'continue', got {self.on_resume!r}.")
        if self.mode not in (None, "online", "offline", "disabled"):
            raise ValueError(f"`wandb.mode` must be 'online', 'offline' or 'disabled', got {self.mode!r}.")

    def to_wandb_kwargs(self, step: int | None = None) -> dict[str, Any]:
        """Keyword arguments for ``wandb.init``.  With a ``run_id`` and a resume ``step``: ``id`` + ``resume="allow"``
        under ``on_resume="continue"``, else ``fork_from="<run>?_step=<step>"`` with a note saying so (offline and
        disabled modes cannot fork on the server: the note records what would have happened)."""
        kw = {k: getattr(self, k) for k in ("entity", "name", "notes", "tags", "group", "job_type", "mode")}
        kw["tags"] = list(kw["tags"])
        if self.run_id is not None and step is not None:
            if self.on_resume == "continue":
                kw["id"], kw["resume"] = self.run_id, "allow"
            else:
                offline = self.mode in ("offline", "disabled")
                note = (f"(offline) would fork from run {self.run_id} at step {step}." if offline
                        else f"Forked from run {self.run_id} at step {step}.")
                if not offline:
                    kw["fork_from"] = f"{self.run_id}?_step={step}"
                kw["notes"] = note if kw.get("notes") is None else f"{kw['notes']}\n{note}"
        return kw


_VIDEO_PRESETS = ("ultrafast", "superfast", "veryfast", "faster", "fast", "medium", "slow", "slower", "veryslow")


@dataclass
class EvalConfig:
    """``seed`` seeds the evaluation environments (falls back to the pipeline seed); ``decorrelate_rank_seeds`` gives
    every rank its own slice of scenes (False: all ranks seed alike, so the evaluation is reproducible across world
    sizes); ``seed_list``: explicit seeds, a list or a comma-separated string, evaluated exactly (their count replaces
    ``n_episodes``).  The ``video_*`` fields shape the uploaded grid-summary video: H.264 quality target (0-51), encoder
    preset, and every how-many-th frame is kept."""

    n_episodes: int = 16
    batch_size: int = 16
    use_async_envs: bool = True
    max_episodes_rendered: int = 16
    grid_size: tuple[int, int] | None = None
    video_fps: int | None = None
    video_crf: int = 30
    video_preset: str = "veryfast"
    video_frame_stride: int = 2
    keep_per_episode_videos: bool = False
    recording_root: str | None = None
    seed: int | None = None
    decorrelate_rank_seeds: bool = False
    goal_frames_dir: str | None = None
    seed_list: Any = None
    dataset_repo_id: str | None = None
    robot_type: str | None = None
    control_mode: str | None = None

    def __post_init__(self):
        if isinstance(self.seed_list, str):
            self.seed_list = [int(x) for x in self.seed_list.split(",") if x.strip() != ""]
        if self.seed_list is not None:
            self.seed_list = [int(x) for x in self.seed_list]
            if not self.seed_list:
                raise ValueError("eval.seed_list is empty")
            self.n_episodes = len(self.seed_list)
            self.batch_size = min(self.batch_size, self.n_episodes)
        if self.batch_size > self.n_episodes:
            raise ValueError(
                f"The eval batch size is greater than the number of eval episodes ({self.batch_size} > "
                f"{self.n_episodes}): {self.batch_size} environments would be instantiated and only {self.n_episodes} "
                f"used. Raise `eval.n_episodes` to {self.batch_size} or lower `eval.batch_size` to {self.n_episodes}.")
        if not 0 <= self.video_crf <= 51:
            raise ValueError(f"eval.video_crf must be in [0, 51], got {self.video_crf}.")
        if self.video_frame_stride < 1:
            raise ValueError(f"eval.video_frame_stride must be >= 1, got {self.video_frame_stride}.")
        if self.video_preset not in _VIDEO_PRESETS:
            raise ValueError(f"eval.video_preset must be one of {sorted(_VIDEO_PRESETS)}, got {self.video_preset!r}.")


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
