"""Environment configurations (``type: fake | libero | robocasa``; reference ``src/opentau/envs/configs.py``).

LIBERO and RoboCasa render through MuJoCo on an OpenGL / EGL context.  No graphics stack exists on these machines,
so their factories raise with that reason; the headless ``fake`` environment has the same observation / action
interface and lets the whole evaluation pipeline (vector envs, rollouts, success accounting, per-task grouping,
metric gathers) run anywhere.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..configs.codec import ChoiceRegistry
from ..configs.types import FeatureType, PolicyFeature


SPEED_BUCKET_STEP = 10
CONTROL_MODE_CHOICES = ("joint", "ee")


@dataclass
class EnvMetadataConfig:
    """Metadata the pi0.7 family tokenizes as a ``"Metadata: ..."`` segment of its prefix, broadcast over the rollout
    batch at inference (reference ``src/opentau/envs/configs.py:46-126``).  It belongs to the environment config (WHAT is
    being run), not the eval config (how much of it).  ``None`` leaves a field out: no batch key, no segment.  Allowed
    values are those the dataset emits in training: ``speed`` a multiple of 10 in [0, 100] (0 = fastest decile of the
    task), ``quality`` in [1, 5], ``mistake`` a bool (``False`` emits "Mistake: False", which differs from leaving it
    out), ``robot_type`` a non-empty string, ``control_mode`` ``"joint"`` or ``"ee"``.  ``emit_fps`` broadcasts the
    environment's stepping frequency as ``fps``; off by default so that checkpoints trained without that conditioning
    see no surprise segment.  Other policy families ignore all of it."""

    speed: int | None = None
    quality: int | None = None
    mistake: bool | None = None
    robot_type: str | None = None
    control_mode: str | None = None
    emit_fps: bool = False

    def __post_init__(self) -> None:
        def is_int(x):            # bool is a subclass of int: speed=True must not pass as 1
            return isinstance(x, int) and not isinstance(x, bool)
        if self.speed is not None:
            if not is_int(self.speed):
                raise TypeError(f"env.metadata.speed must be int, got {type(self.speed).__name__}")
            if not 0 <= self.speed <= 100 or self.speed % SPEED_BUCKET_STEP:
                raise ValueError(f"env.metadata.speed must be a multiple of {SPEED_BUCKET_STEP} in [0, 100], got {self.speed}")
        if self.quality is not None:
            if not is_int(self.quality):
                raise TypeError(f"env.metadata.quality must be int, got {type(self.quality).__name__}")
            if not 1 <= self.quality <= 5:
                raise ValueError(f"env.metadata.quality must be in [1, 5], got {self.quality}")
        if self.mistake is not None and not isinstance(self.mistake, bool):
            raise TypeError(f"env.metadata.mistake must be bool, got {type(self.mistake).__name__}")
        if self.robot_type is not None:
            if not isinstance(self.robot_type, str):
                raise TypeError(f"env.metadata.robot_type must be str, got {type(self.robot_type).__name__}")
            if not self.robot_type:
                raise ValueError("env.metadata.robot_type must be a non-empty string; use None to leave it out")
        if self.control_mode is not None and self.control_mode not in CONTROL_MODE_CHOICES:
            raise ValueError(f"env.metadata.control_mode must be one of {CONTROL_MODE_CHOICES} or None, got "
                             f"{self.control_mode!r}")


@dataclass
class EnvConfig(ChoiceRegistry):
    task: str | None = None
    fps: int = 30
    episode_length: int = 100
    max_parallel_tasks: int = 1
    features: dict[str, PolicyFeature] = field(default_factory=dict)
    features_map: dict[str, str] = field(default_factory=dict)
    metadata: EnvMetadataConfig = field(default_factory=EnvMetadataConfig)

    @property
    def type(self) -> str:
        return self.get_choice_name()

    @property
    def gym_kwargs(self) -> dict:
        return {}


@EnvConfig.register_subclass("fake")
@dataclass
class FakeEnvConfig(EnvConfig):
    """Point-mass reaching task: the state holds position and goal; success = within ``tolerance`` of the goal."""

    task: str | None = "reach"
    tasks: list[str] = field(default_factory=lambda: ["reach the goal"])
    task_groups: dict[str, list[int]] | None = None
    state_dim: int = 8
    action_dim: int = 4
    num_cams: int = 1
    resolution: tuple[int, int] = (64, 64)
    tolerance: float = 0.1
    action_scale: float = 0.25
    episode_length: int = 40

    def __post_init__(self):
        self.features = {"action": PolicyFeature(FeatureType.ACTION, (self.action_dim,)),
                         "agent_pos": PolicyFeature(FeatureType.STATE, (self.state_dim,)),
                         **{f"pixels/camera{i}": PolicyFeature(FeatureType.VISUAL, (*self.resolution, 3))
                            for i in range(self.num_cams)}}
        self.features_map = {"action": "actions", "agent_pos": "state",
                             **{f"pixels/camera{i}": f"camera{i}" for i in range(self.num_cams)}}


@EnvConfig.register_subclass("libero")
@dataclass
class LiberoEnvConfig(EnvConfig):
    task: str | None = "libero_10"
    task_ids: list[int] | None = None
    camera_name: str = "agentview_image,robot0_eye_in_hand_image"
    init_states: bool = True
    episode_length: int = 520
    observation_height: int = 256
    observation_width: int = 256


@EnvConfig.register_subclass("robocasa")
@dataclass
class RoboCasaEnvConfig(EnvConfig):
    task: str | None = "NavigateKitchen"
    episode_length: int = 500
    camera_names: list[str] = field(default_factory=lambda: ["robot0_agentview_left", "robot0_eye_in_hand"])
