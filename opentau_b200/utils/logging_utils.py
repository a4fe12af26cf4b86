"""Metric meters with accumulate-on-assign semantics and rank-0 logging set-up
(reference ``src/opentau/utils/logging_utils.py:29-182``, ``utils/utils.py:170-216``)."""

from __future__ import annotations

import logging
import os
from typing import Any


class AverageMeter:
    """Running average; ``update(val, n)`` adds ``n`` observations of value ``val``."""

    def __init__(self, name: str, fmt: str = ":f"):
        self.name, self.fmt = name, fmt
        self.reset()

    def reset(self) -> None:
        self.val = 0.0
        self.avg = 0.0
        self.sum = 0.0
        self.count = 0.0

    def update(self, val: float, n: float = 1) -> None:
        self.val = val
        self.sum += val * n
        self.count += n
        self.avg = self.sum / self.count if self.count else 0.0

    def __str__(self) -> str:
        return f"{self.name}:{{avg{self.fmt}}}".format(avg=self.avg)


class MetricsTracker:
    """Tracks step / sample / episode / epoch counters and a dict of :class:`AverageMeter`.

    Assigning ``tracker.loss = x`` updates the meter named ``loss``; reading returns the meter.
    """

    __keys__ = ["_batch_size", "_num_frames", "_avg_samples_per_ep", "metrics", "steps", "samples", "episodes",
                "epochs"]

    def __init__(self, batch_size: int, num_frames: int | None = None, num_episodes: int | None = None,
                 metrics: dict[str, AverageMeter] | None = None, initial_step: int = 0):
        self.__dict__.update(dict.fromkeys(self.__keys__))
        self._batch_size = batch_size
        self._num_frames = num_frames or 0
        self._avg_samples_per_ep = (num_frames / num_episodes) if num_frames and num_episodes else 0
        self.metrics = metrics or {}
        self.steps = initial_step
        self.samples = self.steps * batch_size
        self.episodes = self.samples / self._avg_samples_per_ep if self._avg_samples_per_ep else 0
        self.epochs = self.samples / self._num_frames if self._num_frames else 0

    def __getattr__(self, name: str) -> Any:
        if name in self.__dict__:
            return self.__dict__[name]
        if name in self.__dict__.get("metrics", {}):
            return self.__dict__["metrics"][name]
        raise AttributeError(f"'{type(self).__name__}' object has no attribute '{name}'")

    def __setattr__(self, name: str, value: Any) -> None:
        if name in self.__dict__ or name in self.__keys__:
            super().__setattr__(name, value)
        elif name in self.metrics:
            self.metrics[name].update(float(value))
        else:
            raise AttributeError(f"'{type(self).__name__}' object has no attribute '{name}'")

    def step(self) -> None:
        self.steps += 1
        self.samples += self._batch_size
        if self._avg_samples_per_ep:
            self.episodes = self.samples / self._avg_samples_per_ep
        if self._num_frames:
            self.epochs = self.samples / self._num_frames

    def __str__(self) -> str:
        parts = [f"step:{self.steps}", f"smpl:{self.samples}", f"ep:{int(self.episodes)}", f"epch:{self.epochs:.2f}"]
        parts += [str(m) for m in self.metrics.values()]
        return " ".join(parts)

    def to_dict(self, use_avg: bool = True) -> dict[str, float]:
        d = {"steps": self.steps, "samples": self.samples, "episodes": self.episodes, "epochs": self.epochs}
        d.update({k: (m.avg if use_avg else m.val) for k, m in self.metrics.items()})
        return d

    def reset_averages(self) -> None:
        for m in self.metrics.values():
            m.reset()


def init_logging(rank: int = 0, level: int = logging.INFO) -> None:
    """INFO on rank 0, WARNING elsewhere; timestamped single-line records."""
    fmt = logging.Formatter("%(levelname)s %(asctime)s %(filename)s:%(lineno)d %(message)s", "%Y-%m-%d %H:%M:%S")
    root = logging.getLogger()
    for h in list(root.handlers):
        root.removeHandler(h)
    h = logging.StreamHandler()
    h.setFormatter(fmt)
    root.addHandler(h)
    root.setLevel(level if rank == 0 else logging.WARNING)


def format_big_number(num: float, precision: int = 0) -> str:
    for suffix in ["", "K", "M", "B", "T", "Q"]:
        if abs(num) < 1000:
            return f"{num:.{precision}f}{suffix}"
        num /= 1000
    return f"{num:.{precision}f}Q"
