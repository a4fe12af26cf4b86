"""Settings of the ROS 2 bag -> LeRobot conversion (reference ``src/opentau/configs/ros2lerobot.py``)."""

from __future__ import annotations

from dataclasses import dataclass, field

from .types import ROSFeature


@dataclass
class RosToLeRobotConfig:
    input_path: str = "input_path"          # directory with one sub-directory per bag
    output_path: str = "output_path"        # root of the LeRobot dataset to create
    fps: int = 10                           # every topic is resampled to this rate
    joint_order: list[str] = field(default_factory=list)   # empty: taken from the first joint message
    robot_type: str = "unknown"
    dataset_features: dict[str, ROSFeature] = field(default_factory=dict)
