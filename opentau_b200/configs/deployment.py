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

    def __post_init__(self):
        if not (0 < self.port < 65536):
            raise ValueError(f"port out of range: {self.port}")
        if self.max_workers < 1:
            raise ValueError("max_workers must be >= 1")


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
