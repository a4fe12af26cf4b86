"""SO-101 follower arm, leader arm and cameras (reference ``src/opentau/scripts/so101/{robots,teleoperators,cameras}``)."""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

import numpy as np

from .motors_bus import SO101_MOTORS, MotorCalibration, MotorsBus


@dataclass
class CameraConfig:
    index_or_path: int | str = 0
    width: int = 640
    height: int = 480
    fps: int = 30


class OpenCVCamera:
    def __init__(self, cfg: CameraConfig):
        self.cfg, self.cap = cfg, None

    def connect(self) -> None:
        import cv2
        self.cap = cv2.VideoCapture(self.cfg.index_or_path)
        if not self.cap.isOpened():
            raise ConnectionError(f"cannot open camera {self.cfg.index_or_path}")
        self.cap.set(cv2.CAP_PROP_FRAME_WIDTH, self.cfg.width)
        self.cap.set(cv2.CAP_PROP_FRAME_HEIGHT, self.cfg.height)
        self.cap.set(cv2.CAP_PROP_FPS, self.cfg.fps)

    def read(self) -> np.ndarray:
        ok, bgr = self.cap.read()
        if not ok:
            raise IOError(f"camera {self.cfg.index_or_path} returned no frame")
        return np.ascontiguousarray(bgr[:, :, ::-1])

    def disconnect(self) -> None:
        if self.cap is not None:
            self.cap.release()
            self.cap = None

    @staticmethod
    def find_cameras(max_index: int = 10) -> list[dict]:
        import cv2
        found = []
        for i in range(max_index):
            cap = cv2.VideoCapture(i)
            if cap.isOpened():
                found.append({"index": i, "width": int(cap.get(cv2.CAP_PROP_FRAME_WIDTH)),
                              "height": int(cap.get(cv2.CAP_PROP_FRAME_HEIGHT)), "fps": cap.get(cv2.CAP_PROP_FPS)})
            cap.release()
        return found


@dataclass
class SOArmConfig:
    port: Any = "/dev/ttyACM0"
    id: str = "so101"
    calibration_dir: str = "~/.cache/opentau/calibration"
    max_relative_target: float | None = None       # safety clamp on the per-step joint move (normalised units)
    cameras: dict[str, CameraConfig] = field(default_factory=dict)


class _SOArm:
    role = "arm"

    def __init__(self, cfg: SOArmConfig):
        self.cfg = cfg
        self.bus = MotorsBus(cfg.port, SO101_MOTORS)
        self.cameras = {n: OpenCVCamera(c) for n, c in cfg.cameras.items()}

    @property
    def calibration_path(self) -> Path:
        return Path(self.cfg.calibration_dir).expanduser() / self.role / f"{self.cfg.id}.json"

    @property
    def is_calibrated(self) -> bool:
        return bool(self.bus.calibration)

    def connect(self, calibrate: bool = False) -> None:
        self.bus.connect()
        if self.calibration_path.exists():
            self.bus.load_calibration(self.calibration_path)
        elif calibrate:
            self.calibrate()
        for c in self.cameras.values():
            c.connect()
        self.configure()

    def configure(self) -> None:
        pass

    def calibrate(self, ranges: dict[str, tuple[int, int]] | None = None) -> dict[str, MotorCalibration]:
        """Half-turn homing at the current (mid-range) pose, then the joint ranges: given, or recorded while the
        operator moves every joint through its travel until Enter is pressed."""
        self.bus.disable_torque()
        homing = self.bus.set_half_turn_homings()
        if ranges is None:
            ranges = self._record_ranges()
        cal = {n: MotorCalibration(m.id, 0, homing[n], int(ranges[n][0]), int(ranges[n][1])) for n, m in self.bus.motors.items()}
        self.bus.write_calibration(cal)
        self.bus.save_calibration(self.calibration_path)
        return cal

    def _record_ranges(self) -> dict[str, tuple[int, int]]:  # pragma: no cover - interactive
        import select
        import sys
        print("Move every joint through its full range, then press Enter.")
        lo = hi = None
        while True:
            pos = self.bus.sync_read("Present_Position", normalize=False)
            lo = pos if lo is None else {k: min(lo[k], v) for k, v in pos.items()}
            hi = pos if hi is None else {k: max(hi[k], v) for k, v in pos.items()}
            if select.select([sys.stdin], [], [], 0.02)[0]:
                sys.stdin.readline()
                break
        return {k: (int(lo[k]), int(hi[k])) for k in lo}

    def disconnect(self) -> None:
        self.bus.disconnect()
        for c in self.cameras.values():
            c.disconnect()


class SOFollower(_SOArm):
    role = "robots"

    def configure(self) -> None:
        self.bus.disable_torque()
        self.bus.configure_motors()
        self.bus.enable_torque()

    def get_observation(self) -> dict[str, Any]:
        obs = {f"{n}.pos": v for n, v in self.bus.sync_read("Present_Position").items()}
        for n, c in self.cameras.items():
            obs[n] = c.read()
        return obs

    def send_action(self, action: dict[str, float]) -> dict[str, float]:
        goal = {k.removesuffix(".pos"): float(v) for k, v in action.items()}
        m = self.cfg.max_relative_target
        if m is not None:
            cur = self.bus.sync_read("Present_Position")
            goal = {k: cur[k] + min(max(v - cur[k], -m), m) for k, v in goal.items()}
        self.bus.sync_write("Goal_Position", goal)
        return {f"{k}.pos": v for k, v in goal.items()}


class SOLeader(_SOArm):
    role = "teleoperators"

    def configure(self) -> None:
        self.bus.disable_torque()

    def get_action(self) -> dict[str, float]:
        return {f"{n}.pos": v for n, v in self.bus.sync_read("Present_Position").items()}


@dataclass
class BiSOArmConfig:
    """Two SO arms driven as one device (reference ``src/opentau/scripts/so101/robots/bi_so_follower/
    config_bi_so_follower.py:21-31`` and ``teleoperators/bi_so_leader/config_bi_so_leader.py``)."""
    left: SOArmConfig = field(default_factory=SOArmConfig)
    right: SOArmConfig = field(default_factory=lambda: SOArmConfig(port="/dev/ttyACM1"))
    id: str | None = None
    calibration_dir: str | None = None


class _BiSOArm:
    """Pair of arms; every key of the pair is the single arm's key with a ``left_`` / ``right_`` prefix, and each
    side keeps its own calibration file ``<id>_left`` / ``<id>_right`` (reference ``bi_so_follower.py:33-159``,
    ``bi_so_leader.py:30-118``)."""
    arm_cls: type = _SOArm

    def __init__(self, cfg: BiSOArmConfig):
        from dataclasses import replace
        self.cfg = cfg
        sides = {}
        for side in ("left", "right"):
            c: SOArmConfig = getattr(cfg, side)
            sides[side] = self.arm_cls(replace(
                c, id=f"{cfg.id}_{side}" if cfg.id else c.id,
                calibration_dir=cfg.calibration_dir if cfg.calibration_dir else c.calibration_dir))
        self.left_arm, self.right_arm = sides["left"], sides["right"]
        self.cameras = {**{f"left_{n}": c for n, c in self.left_arm.cameras.items()},
                        **{f"right_{n}": c for n, c in self.right_arm.cameras.items()}}

    @property
    def arms(self):
        return (("left", self.left_arm), ("right", self.right_arm))

    @property
    def is_calibrated(self) -> bool:
        return all(a.is_calibrated for _, a in self.arms)

    def connect(self, calibrate: bool = False) -> None:
        for _, a in self.arms:
            a.connect(calibrate)

    def configure(self) -> None:
        for _, a in self.arms:
            a.configure()

    def calibrate(self, ranges: dict[str, dict[str, tuple[int, int]]] | None = None) -> dict:
        return {side: a.calibrate(None if ranges is None else ranges[side]) for side, a in self.arms}

    def disconnect(self) -> None:
        for _, a in self.arms:
            a.disconnect()

    @staticmethod
    def _split(values: dict[str, Any]) -> dict[str, dict[str, Any]]:
        out: dict[str, dict[str, Any]] = {"left": {}, "right": {}}
        for k, v in values.items():
            for side in out:
                if k.startswith(side + "_"):
                    out[side][k[len(side) + 1:]] = v
        return out


class BiSOFollower(_BiSOArm):
    arm_cls = SOFollower

    def get_observation(self) -> dict[str, Any]:
        return {f"{side}_{k}": v for side, a in self.arms for k, v in a.get_observation().items()}

    def send_action(self, action: dict[str, float]) -> dict[str, float]:
        parts = self._split(action)
        return {f"{side}_{k}": v for side, a in self.arms for k, v in a.send_action(parts[side]).items()}


class BiSOLeader(_BiSOArm):
    arm_cls = SOLeader

    def get_action(self) -> dict[str, float]:
        return {f"{side}_{k}": v for side, a in self.arms for k, v in a.get_action().items()}


def teleoperate_step(leader, follower) -> tuple[dict, dict]:
    action = leader.get_action()
    sent = follower.send_action(action)
    return follower.get_observation(), sent


def busy_wait(seconds: float) -> None:
    end = time.perf_counter() + seconds
    while time.perf_counter() < end:
        pass
