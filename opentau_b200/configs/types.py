"""Feature / normalization enums and the policy feature record.

Same names and values as the reference schema (OpenTau ``src/opentau/configs/types.py:29-106``) so
that ``config.json`` files stay interchangeable.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum


class FeatureType(str, Enum):
    STATE = "STATE"
    VISUAL = "VISUAL"
    ENV = "ENV"
    ACTION = "ACTION"


class NormalizationMode(str, Enum):
    MIN_MAX = "MIN_MAX"
    MEAN_STD = "MEAN_STD"
    QUANTILE = "QUANTILE"   # [q01, q99] -> [-1, 1], falling back to min/max where quantiles are absent
    IDENTITY = "IDENTITY"


@dataclass
class PolicyFeature:
    type: FeatureType
    shape: tuple


@dataclass
class ROSFeature:
    ros_topic: str
    topic_attribute: str
    enum_values: str
    dtype: str
    shape: tuple
