"""General helpers (reference ``src/opentau/utils/utils.py:60-490``)."""

from __future__ import annotations

import logging
import os
import platform
import subprocess
from datetime import datetime, timezone
from pathlib import Path
from typing import Any

import numpy as np
import torch

from .logging_utils import format_big_number, init_logging  # noqa: F401  (re-exported like the reference module)


def none_or_int(value: str) -> int | None:
    return None if value == "None" else int(value)


def inside_slurm() -> bool:
    return "SLURM_JOB_ID" in os.environ


def auto_torch_device() -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda")
    return torch.device("cpu")


def auto_select_torch_device() -> torch.device:
    dev = auto_torch_device()
    logging.info("%s backend detected, using %s.", "Cuda" if dev.type == "cuda" else "No accelerated", dev)
    return dev


def get_safe_torch_device(try_device: str, log: bool = False) -> torch.device:
    dev = torch.device(try_device)
    if dev.type == "cuda" and not torch.cuda.is_available():
        raise AssertionError("CUDA was requested but is not available")
    if log and dev.type != "cuda":
        logging.warning("Using %s: expect this to be much slower than a B200.", dev)
    return dev


def get_safe_dtype(dtype: torch.dtype, device: str | torch.device) -> torch.dtype:
    return dtype


def is_torch_device_available(try_device: str) -> bool:
    if try_device == "cuda":
        return torch.cuda.is_available()
    if try_device == "cpu":
        return True
    raise ValueError(f"Unknown device '{try_device}'.")


def is_amp_available(device: str) -> bool:
    if device in ("cuda", "cpu"):
        return True
    raise ValueError(f"Unknown device '{device}'.")


def is_valid_numpy_dtype_string(dtype_str: str) -> bool:
    try:
        np.dtype(dtype_str)
        return True
    except TypeError:
        return False


def capture_timestamp_utc() -> datetime:
    return datetime.now(timezone.utc)


def say(text: str, blocking: bool = False) -> None:
    """Spoken feedback for teleoperation on a desktop; a log line elsewhere."""
    logging.info("[say] %s", text)


def log_say(text: str, play_sounds: bool, blocking: bool = False) -> None:
    logging.info(text)
    if play_sounds:
        say(text, blocking)


def get_git_commit_hash() -> str | None:
    try:
        return subprocess.check_output(["git", "rev-parse", "HEAD"], stderr=subprocess.DEVNULL).decode().strip()
    except Exception:  # noqa: BLE001
        return None


def has_method(obj: object, name: str) -> bool:
    return callable(getattr(obj, name, None))


def create_dummy_observation(cfg, device, dtype: torch.dtype = torch.float32, batch_size: int = 1) -> dict[str, Any]:
    """A random observation of the pipeline's shapes: ``camera{i}``, ``state``, ``prompt`` and pad masks."""
    H, W = cfg.resolution
    obs: dict[str, Any] = {f"camera{i}": torch.rand(batch_size, 3, H, W, device=device, dtype=dtype)
                           for i in range(cfg.num_cams)}
    obs["state"] = torch.zeros(batch_size, cfg.max_state_dim, device=device, dtype=dtype)
    obs["prompt"] = ["Pick up yellow lego block and put it in the bin"] * batch_size
    obs["img_is_pad"] = torch.zeros(batch_size, cfg.num_cams, dtype=torch.bool, device=device)
    obs["action_is_pad"] = torch.zeros(batch_size, cfg.action_chunk, dtype=torch.bool, device=device)
    return obs


def on_main_process(fn, *args, sync: bool = True, **kwargs):
    """Runs ``fn`` on rank 0 and (optionally) hands its result to every rank."""
    from ..parallel import control
    return control.on_main_process(fn, *args, sync=sync, **kwargs)


def display_sys_info() -> dict[str, str]:
    info = {"python": platform.python_version(), "platform": platform.platform(), "torch": torch.__version__,
            "cuda": str(torch.version.cuda), "gpus": str(torch.cuda.device_count())}
    for k, v in info.items():
        print(f"{k:10s} {v}")
    return info
