"""Single-task LIBERO evaluation settings attached to a training config (reference ``src/opentau/configs/libero.py``).

``suite`` is one of ``spatial | object | goal | 10 | 90``, ``id`` the task index inside it; ``chunk_usage`` (how many
actions of each predicted chunk are executed before the next observation) defaults to the training config's
``action_chunk`` and must lie in ``1 .. action_chunk``.  The reference resolves the task's BDDL file and initial states
at construction through the simulator package; here that lookup is deferred to ``envs.libero.real_backend()`` so the
config can be built, validated and serialised on a machine without the simulator.
"""

from __future__ import annotations

from dataclasses import dataclass

from .train import TrainPipelineConfig

SUITE_SIZES = {"spatial": 10, "object": 10, "goal": 10, "10": 10, "90": 90}


@dataclass
class LiberoEnvConfig:
    suite: str = "10"
    id: int = 0
    max_steps: int = 1000
    chunk_usage: int | None = None
    n_simulations: int = 100
    video_dir: str | None = None

    def __post_init__(self):
        self.suite = str(self.suite).lower().removeprefix("libero_")
        if self.suite not in SUITE_SIZES:
            raise ValueError(f"Invalid suite {self.suite!r}. Available suites are: {sorted(SUITE_SIZES)}")
        if not 0 <= self.id < SUITE_SIZES[self.suite]:
            raise ValueError(f"Invalid task id {self.id} for suite {self.suite!r}: ids run from 0 to "
                             f"{SUITE_SIZES[self.suite] - 1}")

    @property
    def suite_name(self) -> str:
        return f"libero_{self.suite}"


@dataclass
class TrainConfigWithLiberoEval(TrainPipelineConfig):
    libero: LiberoEnvConfig | None = None

    def __post_init__(self):
        super().__post_init__()
        if self.libero is None:
            raise ValueError("Libero config must be provided.")
        if isinstance(self.libero, dict):
            self.libero = LiberoEnvConfig(**self.libero)
        if self.libero.chunk_usage is None:
            self.libero.chunk_usage = self.action_chunk
        if not 1 <= self.libero.chunk_usage <= self.action_chunk:
            raise ValueError(f"chunk_usage must be between 1 and action_chunk={self.action_chunk}, "
                             f"got {self.libero.chunk_usage}")
