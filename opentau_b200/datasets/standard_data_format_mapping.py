"""Raw feature name -> standard name tables per dataset (reference
``src/opentau/datasets/standard_data_format_mapping.py:20-290``).

A mapping goes from the standard key (``camera0``, ``state``, ``actions``, ``prompt``, ``response`` ...) to the
dataset's column.  Datasets absent from the table fall back to :func:`infer_mapping`, which picks image features in
sorted order and the conventional LeRobot names.
"""

from __future__ import annotations

DATA_FEATURES_NAME_MAPPING: dict[str, dict[str, str]] = {
    "lerobot/aloha_mobile_cabinet": {"camera0": "observation.images.cam_high", "camera1": "observation.images.cam_left_wrist",
                                     "camera2": "observation.images.cam_right_wrist", "state": "observation.state",
                                     "actions": "action", "prompt": "task", "response": "response"},
    "lerobot/droid_100": {"camera0": "observation.images.exterior_image_1_left",
                          "camera1": "observation.images.wrist_image_left", "state": "observation.state",
                          "actions": "action", "prompt": "task", "response": "response"},
    "physical-intelligence/libero": {"camera0": "image", "camera1": "wrist_image", "state": "state",
                                     "actions": "actions", "prompt": "task", "response": "response"},
    "lerobot/libero": {"camera0": "observation.images.image", "camera1": "observation.images.wrist_image",
                       "state": "observation.state", "actions": "action", "prompt": "task", "response": "response"},
    "lerobot/pusht": {"camera0": "observation.image", "state": "observation.state", "actions": "action",
                      "prompt": "task", "response": "response"},
}

LOSS_TYPE_MAPPING: dict[str, str] = {}


def infer_mapping(features: dict[str, dict]) -> dict[str, str]:
    cams = sorted(k for k, ft in features.items() if ft["dtype"] in ("image", "video") and "subgoal" not in k)
    m = {f"camera{i}": k for i, k in enumerate(cams)}
    for std, cands in (("state", ("observation.state", "state")), ("actions", ("action", "actions"))):
        for c in cands:
            if c in features:
                m[std] = c
                break
    m["prompt"], m["response"] = "task", "response"
    for opt in ("speed", "quality", "mistake", "memory", "next_memory", "advantage", "success"):
        if opt in features:
            m[opt] = opt
    return m


def get_mapping(repo_id: str, features: dict[str, dict], override: dict[str, str] | None = None) -> dict[str, str]:
    if override:
        return dict(override)
    if repo_id in DATA_FEATURES_NAME_MAPPING:
        return dict(DATA_FEATURES_NAME_MAPPING[repo_id])
    return infer_mapping(features)
