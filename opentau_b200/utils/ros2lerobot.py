"""Feature extractors and time alignment for ROS 2 messages (reference ``src/opentau/utils/ros2lerobot.py:31-245``).

An extractor turns one deserialised message into the value of a dataset feature: joint state (positions then
velocities, in the configured joint order; joints missing from the message read 0), joint action (the ``q`` field of the
per-joint commands), or an image (compressed bytes decoded to HxWx3 RGB).  Messages are plain attribute objects, so the
code runs on anything shaped like them; the ``rosbags`` reader is needed only to pull them out of a bag file.
"""

from __future__ import annotations

import io
import logging
from typing import Any

import numpy as np


def get_nested_item(obj: Any, flattened_key: str, sep: str = ".") -> Any:
    for key in flattened_key.split(sep):
        obj = getattr(obj, key)
    return obj


def stamp_to_sec(ts: Any) -> float:
    """A ``builtin_interfaces/Time``-like object, or integer nanoseconds as a bag reader reports them."""
    if hasattr(ts, "sec"):
        return ts.sec + ts.nanosec / 1e9
    return float(ts) / 1e9


class FeatureExtractor:
    def __init__(self, cfg):
        self.cfg = cfg

    def _order(self, names) -> list[str]:
        if not self.cfg.joint_order:
            self.cfg.joint_order = list(names)
            logging.info("joint order taken from the first message: %s", self.cfg.joint_order)
        return self.cfg.joint_order


class StateExtractor(FeatureExtractor):
    def __call__(self, msg: Any, topic: str, attribute: str) -> list[float]:
        if not hasattr(msg, "name"):
            return []
        try:
            where = {n: i for i, n in enumerate(msg.name)}
            pos, vel = get_nested_item(msg, attribute), get_nested_item(msg, "velocity")
            pick = lambda arr, n: float(arr[where[n]]) if n in where and len(arr) > where[n] else 0.0  # noqa: E731
            order = self._order(msg.name)
            return [pick(pos, n) for n in order] + [pick(vel, n) for n in order]
        except (KeyError, AttributeError, TypeError) as e:
            logging.warning("could not read %s from %s: %s", attribute, topic, e)
            return []


class ActionExtractor(FeatureExtractor):
    def __call__(self, msg: Any, topic: str, attribute: str) -> list[float]:
        if not hasattr(msg, "joint_names"):
            return []
        try:
            where = {n: i for i, n in enumerate(msg.joint_names)}
            q = [c.q for c in get_nested_item(msg, attribute)]
            return [float(q[where[n]]) if n in where and len(q) > where[n] else 0.0
                    for n in self._order(msg.joint_names)]
        except (KeyError, AttributeError, TypeError) as e:
            logging.warning("could not read %s from %s: %s", attribute, topic, e)
            return []


class ImageExtractor(FeatureExtractor):
    def __call__(self, msg: Any, topic: str, attribute: str):
        try:
            from PIL import Image
            img = np.array(Image.open(io.BytesIO(bytes(get_nested_item(msg, attribute)))))
            if img.ndim == 2:
                img = np.stack([img] * 3, -1)
            return img[..., :3]
        except Exception as e:  # noqa: BLE001 - a broken frame is skipped, not fatal
            logging.warning("could not decode the image on %s: %s", topic, e)
            return None


EXTRACTORS = {"state": StateExtractor, "action": ActionExtractor, "image": ImageExtractor}


def synchronize_sensor_data(data: list[tuple[Any, Any]], fps: int, start_time: float) -> list[Any]:
    """Resamples one ``(stamp, value)`` stream (ascending stamps) to ``fps`` from ``start_time``: frame 0 is the first
    sample, frame ``i`` the sample nearest to ``start + i / fps``; the number of frames is
    ``int((last stamp - start) * fps)``."""
    if not data:
        return []
    times = [stamp_to_sec(t) for t, _ in data]
    out, idx = [data[0][1]], 0
    for frame in range(1, int((times[-1] - start_time) * fps)):
        now = start_time + frame / fps
        while idx < len(data) - 1 and abs(now - times[idx]) > abs(now - times[idx + 1]):
            idx += 1
        out.append(data[idx][1])
    return out
