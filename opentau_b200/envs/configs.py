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


@dataclass
class EnvConfig(ChoiceRegistry):
    task: str | None = None
    fps: int = 30
    episode_length: int = 100
    max_parallel_tasks: int = 1
    features: dict[str, PolicyFeature] = field(default_factory=dict)
    features_map: dict[str, str] = field(default_factory=dict)

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
