"""Named-motor bus with calibration and unit conversion (reference ``src/opentau/scripts/so101/motors/motors_bus.py``).

Positions are exposed normalised: ``RANGE_M100_100`` maps the calibrated ``[range_min, range_max]`` to ``[-100, 100]``,
``RANGE_0_100`` (the gripper) to ``[0, 100]``, ``DEGREES`` to degrees about the middle of the range.
"""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass
from enum import Enum
from pathlib import Path

from .feetech import RESOLUTION, FeetechProtocol


class MotorNormMode(str, Enum):
    RANGE_0_100 = "range_0_100"
    RANGE_M100_100 = "range_m100_100"
    DEGREES = "degrees"


@dataclass
class Motor:
    id: int
    model: str = "sts3215"
    norm_mode: MotorNormMode = MotorNormMode.RANGE_M100_100


@dataclass
class MotorCalibration:
    id: int
    drive_mode: int
    homing_offset: int
    range_min: int
    range_max: int


SO101_MOTORS = {"shoulder_pan": Motor(1), "shoulder_lift": Motor(2), "elbow_flex": Motor(3), "wrist_flex": Motor(4),
                "wrist_roll": Motor(5), "gripper": Motor(6, norm_mode=MotorNormMode.RANGE_0_100)}


class MotorsBus:
    def __init__(self, port, motors: dict[str, Motor] | None = None, calibration: dict[str, MotorCalibration] | None = None):
        """``port``: a device path (opened with pyserial at 1 Mbaud) or a transport object."""
        self.motors = dict(motors or SO101_MOTORS)
        self.calibration = dict(calibration or {})
        self._port_arg, self.port, self.proto = port, None, None

    # -- connection -----------------------------------------------------------------------------------
    def connect(self) -> None:
        if isinstance(self._port_arg, str):
            try:
                import serial
            except ImportError as e:
                raise RuntimeError("pyserial is needed to open a serial device") from e
            self.port = serial.Serial(self._port_arg, baudrate=1_000_000, timeout=0.05)
        else:
            self.port = self._port_arg
        self.proto = FeetechProtocol(self.port)
        missing = [n for n, m in self.motors.items() if not self.proto.ping(m.id)]
        if missing:
            raise ConnectionError(f"motors not answering on the bus: {missing}")

    def disconnect(self, disable_torque: bool = True) -> None:
        if self.proto is not None and disable_torque:
            self.disable_torque()
        if self.port is not None and hasattr(self.port, "close"):
            self.port.close()
        self.port = self.proto = None

    @property
    def is_connected(self) -> bool:
        return self.proto is not None

    # -- torque / modes ---------------------------------------------------------------------------------
    def enable_torque(self, names: list[str] | None = None) -> None:
        for n in names or self.motors:
            self.proto.write(self.motors[n].id, "Torque_Enable", 1)
            self.proto.write(self.motors[n].id, "Lock", 1)

    def disable_torque(self, names: list[str] | None = None) -> None:
        for n in names or self.motors:
            self.proto.write(self.motors[n].id, "Torque_Enable", 0)
            self.proto.write(self.motors[n].id, "Lock", 0)

    def configure_motors(self, p: int = 16, i: int = 0, d: int = 32) -> None:
        """Lower P than the factory default avoids shakiness; no return delay; full acceleration."""
        for m in self.motors.values():
            self.proto.write(m.id, "Return_Delay_Time", 0)
            self.proto.write(m.id, "Maximum_Acceleration", 254)
            self.proto.write(m.id, "Acceleration", 254)
            self.proto.write(m.id, "Operating_Mode", 0)
            self.proto.write(m.id, "P_Coefficient", p)
            self.proto.write(m.id, "I_Coefficient", i)
            self.proto.write(m.id, "D_Coefficient", d)

    # -- calibration ------------------------------------------------------------------------------------
    def set_half_turn_homings(self) -> dict[str, int]:
        """With the arm held at the middle of its ranges: choose offsets so that every motor reads half a turn."""
        out = {}
        for n, m in self.motors.items():
            self.proto.write(m.id, "Homing_Offset", 0)
            pos = self.proto.read(m.id, "Present_Position")
            out[n] = pos - (RESOLUTION // 2 - 1)
            self.proto.write(m.id, "Homing_Offset", out[n])
        return out

    def write_calibration(self, calibration: dict[str, MotorCalibration]) -> None:
        for n, c in calibration.items():
            mid = self.motors[n].id
            self.proto.write(mid, "Homing_Offset", c.homing_offset)
            self.proto.write(mid, "Min_Position_Limit", c.range_min)
            self.proto.write(mid, "Max_Position_Limit", c.range_max)
        self.calibration = dict(calibration)

    def save_calibration(self, path: str | Path) -> None:
        Path(path).parent.mkdir(parents=True, exist_ok=True)
        Path(path).write_text(json.dumps({n: asdict(c) for n, c in self.calibration.items()}, indent=2))

    def load_calibration(self, path: str | Path) -> None:
        self.calibration = {n: MotorCalibration(**c) for n, c in json.loads(Path(path).read_text()).items()}

    # -- normalised IO ----------------------------------------------------------------------------------
    def _normalize(self, name: str, raw: int) -> float:
        c, mode = self.calibration.get(name), self.motors[name].norm_mode
        if c is None:
            return float(raw)
        lo, hi = c.range_min, c.range_max
        if hi == lo:
            raise ValueError(f"motor {name}: calibrated range is empty")
        x = min(max(raw, lo), hi)
        if mode is MotorNormMode.RANGE_M100_100:
            v = ((x - lo) / (hi - lo)) * 200.0 - 100.0
            return -v if c.drive_mode else v
        if mode is MotorNormMode.RANGE_0_100:
            v = ((x - lo) / (hi - lo)) * 100.0
            return 100.0 - v if c.drive_mode else v
        return (x - (lo + hi) / 2) * 360.0 / (RESOLUTION - 1)

    def _unnormalize(self, name: str, val: float) -> int:
        c, mode = self.calibration.get(name), self.motors[name].norm_mode
        if c is None:
            return int(round(val))
        lo, hi = c.range_min, c.range_max
        if mode is MotorNormMode.RANGE_M100_100:
            v = -val if c.drive_mode else val
            raw = (min(max(v, -100.0), 100.0) + 100.0) / 200.0 * (hi - lo) + lo
        elif mode is MotorNormMode.RANGE_0_100:
            v = 100.0 - val if c.drive_mode else val
            raw = min(max(v, 0.0), 100.0) / 100.0 * (hi - lo) + lo
        else:
            raw = val * (RESOLUTION - 1) / 360.0 + (lo + hi) / 2
        return int(round(min(max(raw, lo), hi)))

    def sync_read(self, register: str, normalize: bool = True) -> dict[str, float]:
        ids = [m.id for m in self.motors.values()]
        raw = self.proto.sync_read(register, ids)
        names = {m.id: n for n, m in self.motors.items()}
        positional = register in ("Present_Position", "Goal_Position")
        return {names[i]: (self._normalize(names[i], v) if normalize and positional else float(v)) for i, v in raw.items()}

    def sync_write(self, register: str, values: dict[str, float], normalize: bool = True) -> None:
        positional = register in ("Present_Position", "Goal_Position")
        self.proto.sync_write(register, {self.motors[n].id: (self._unnormalize(n, v) if normalize and positional
                                                             else int(round(v))) for n, v in values.items()})
