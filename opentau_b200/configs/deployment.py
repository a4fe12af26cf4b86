"""Serving configuration: gRPC policy server and optional high-level planner
(reference ``src/opentau/configs/deployment.py:49-153``)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class ServerConfig:
    port: int = 50051
    max_workers: int = 4
    max_send_message_length_mb: int = 100
    max_receive_message_length_mb: int = 100
    api_key: str | None = None
    api_key_env: str = "TUNER_INFERENCE_API_KEY"
    use_cuda_graph: bool = True
    warmup_requests: int = 2
    # Which normalisation head serves the requests: both `robot_type` and `control_mode` (the head's key; preferred
    # for multi-head checkpoints) or `dataset_repo_id` (a training dataset name, mapped through the checkpoint's
    # dataset table).  The pair wins when all are set.  All None: a single-head policy uses its only head, a
    # multi-head policy refuses the request.
    dataset_repo_id: str | None = None
    robot_type: str | None = None
    control_mode: str | None = None

    def __post_init__(self):
        if not (0 < self.port < 65536):
            raise ValueError(f"`port` must be between 1 and 65535, got {self.port}.")
        if self.max_workers < 1:
            raise ValueError(f"`max_workers` must be at least 1, got {self.max_workers}.")
        for name in ("max_send_message_length_mb", "max_receive_message_length_mb"):
            if getattr(self, name) < 1:
                raise ValueError(f"`{name}` must be at least 1, got {getattr(self, name)}.")


def tag_norm_head(batch: dict, section) -> dict:
    """Writes the head identity of an eval / server config section (``robot_type`` + ``control_mode``, else
    ``dataset_repo_id``) into an inference batch, in place; nothing when the section names none
    (reference ``src/opentau/scripts/eval.py:203-216``, ``scripts/grpc/server.py:470-487``)."""
    rt, cm = getattr(section, "robot_type", None), getattr(section, "control_mode", None)
    if rt is not None and cm is not None:
        batch["robot_type"], batch["control_mode"] = rt, cm
    elif getattr(section, "dataset_repo_id", None) is not None:
        batch["dataset_repo_id"] = section.dataset_repo_id
    return batch


@dataclass
class PlannerConfig:
    enable: bool = False
    kind: str = "none"            # none | gpt | gemini | open_source
    model: str | None = None
    interval_s: float = 2.0
    memory_max_tokens: int = 256
    prompts_path: str | None = None

    def __post_init__(self):
        if self.kind not in ("none", "gpt", "gemini", "open_source"):
            raise ValueError(f"unknown planner kind {self.kind!r}")
