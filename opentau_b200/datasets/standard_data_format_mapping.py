"""Raw feature name -> standard name tables per dataset (reference
``src/opentau/datasets/standard_data_format_mapping.py:20-290``).

A mapping goes from the standard key (``camera0``, ``state``, ``actions``, ``prompt``, ``response`` ...) to the
dataset's column.  Datasets absent from the table fall back to :func:`infer_mapping`, which picks image features in
sorted order and the conventional LeRobot names.
"""

from __future__ import annotations

#: standard name -> the dataset's column, per repository (``camera{i}``, ``state``, ``actions``, ``prompt``, ``response``;
#: optionally ``mistake`` = a per-frame column of mistakes, ``success`` = a frame column or per-episode outcome that is
#: inverted into ``mistake`` when no mistake column exists and also drives the value model's return bins).  A repository
#: exposed under two control modes registers ``"<repo>::<control_mode>"`` keys (:func:`feature_mapping_key`).
DATA_FEATURES_NAME_MAPPING: dict[str, dict[str, str]] = {
    "ML-GOD/libero": {"camera0": "image", "camera1": "wrist_image", "state": "state", "actions": "actions", "prompt":
        "task", "response": "response"},
    "ML-GOD/libero_spatial_no_noops_1.0.0_lerobot": {"camera0": "observation.images.image", "camera1":
        "observation.images.wrist_image", "state": "observation.state", "actions": "action", "prompt": "task",
        "response": "response"},
    "ML-GOD/mt-button-press": {"camera0": "observation.image", "state": "observation.robot_state", "actions":
        "action", "prompt": "task", "response": "response"},
    "TensorAuto/libero": {"camera0": "image", "camera1": "wrist_image", "state": "state", "actions": "actions",
        "prompt": "task", "response": "response"},
    "autox/agibot-sample": {"camera0": "observation.images.head_left_fisheye", "camera1":
        "observation.images.head_right_fisheye", "camera2": "observation.images.top_head", "camera3":
        "observation.images.hand_left", "camera4": "observation.images.hand_right", "camera5":
        "observation.images.head_center_fisheye", "camera6": "observation.images.back_left_fisheye", "camera7":
        "observation.images.back_right_fisheye", "camera8": "observation.images.cam_top_depth", "state":
        "observation.state", "actions": "action", "prompt": "task", "response": "response"},
    "bi-so100-block-manipulation": {"camera0": "observation.images.top", "camera1": "observation.images.main",
        "camera2": "observation.images.cv", "state": "observation.state", "actions": "action", "prompt": "task",
        "response": "response"},
    "clevr": {"camera0": "image", "state": "state", "actions": "actions", "prompt": "prompt", "response": "postfix"},
    "cocoqa": {"camera0": "image", "state": "state", "actions": "actions", "prompt": "prompt", "response": "postfix"},
    "cube-on-cylinder": {"camera0": "observation.images.top", "camera1": "observation.images.main", "camera2":
        "observation.images.cv", "state": "observation.state", "actions": "action", "prompt": "task", "response":
        "response"},
    "cylinder-on-cube": {"camera0": "observation.images.top", "camera1": "observation.images.main", "camera2":
        "observation.images.cv", "state": "observation.state", "actions": "action", "prompt": "task", "response":
        "response"},
    "danaaubakirova/koch_test": {"camera0": "observation.images.laptop", "camera1": "observation.images.phone",
        "state": "observation.state", "actions": "action", "prompt": "task", "response": "response"},
    "dummy": {"camera0": "image", "state": "state", "actions": "actions", "prompt": "prompt", "response": "postfix"},
    "l-shape-on-cross-shape": {"camera0": "observation.images.top", "camera1": "observation.images.main", "camera2":
        "observation.images.cv", "state": "observation.state", "actions": "action", "prompt": "task", "response":
        "response"},
    "lerobot/aloha_mobile_cabinet": {"camera0": "observation.images.cam_right_wrist", "camera1":
        "observation.images.cam_high", "camera2": "observation.images.cam_left_wrist", "state": "observation.state",
        "actions": "action", "prompt": "task", "response": "response"},
    "lerobot/droid_100": {"camera0": "observation.images.exterior_image_1_left", "camera1":
        "observation.images.exterior_image_2_left", "camera2": "observation.images.wrist_image_left", "state":
        "observation.state", "actions": "action", "prompt": "task", "response": "response"},
    "lerobot/libero": {"camera0": "observation.images.image", "camera1": "observation.images.wrist_image", "state":
        "observation.state", "actions": "action", "prompt": "task", "response": "response"},
    "lerobot/pusht": {"camera0": "observation.image", "state": "observation.state", "actions": "action", "prompt":
        "task", "response": "response"},
    "lerobot/svla_so100_pickplace": {"camera0": "observation.images.top", "camera1": "observation.images.wrist",
        "state": "observation.state", "actions": "action", "prompt": "task", "response": "response"},
    "lerobot/svla_so100_stacking": {"camera0": "observation.images.top", "camera1": "observation.images.wrist",
        "state": "observation.state", "actions": "action", "prompt": "task", "response": "response"},
    "lerobot/svla_so101_pickplace": {"camera0": "observation.images.up", "camera1": "observation.images.side",
        "state": "observation.state", "actions": "action", "prompt": "task", "response": "response"},
    "lerobot_dummy": {"camera0": "camera0", "state": "state", "actions": "actions", "prompt": "task", "response":
        "response"},
    "physical-intelligence/libero": {"camera0": "image", "camera1": "wrist_image", "state": "state", "actions":
        "actions", "prompt": "task", "response": "response"},
    "vsr": {"camera0": "image", "state": "state", "actions": "actions", "prompt": "prompt", "response": "postfix"},
}

#: loss family per dataset: action regression ("MSE") or text targets only ("CE": question-answer corpora)
LOSS_TYPE_MAPPING: dict[str, str] = {
}

_MISSING_CONTROL_MODE_VALUES = frozenset({"unknown"})


def feature_mapping_key(repo_id: str, control_mode: str | None) -> str:
    """``"<repo_id>::<control_mode>"`` for a real control mode, the plain ``repo_id`` otherwise (missing, blank, "unknown").

    Two mixture entries may share a repository and differ in their mapping: one robot exposed as ``joint``
    (``actions -> action_joint``) and as ``ee`` (``actions -> action_ee``).  Keyed by the repository alone the second
    registration would replace the first and the joint entry would silently read the end-effector column
    (reference ``src/opentau/datasets/standard_data_format_mapping.py:254-290``)."""
    cm = (control_mode or "").strip()
    return f"{repo_id}::{cm}" if cm and cm.casefold() not in _MISSING_CONTROL_MODE_VALUES else repo_id


def register_mapping(repo_id: str, mapping: dict[str, str], control_mode: str | None = None) -> str:
    """Adds (or replaces) an entry; returns the key it was stored under."""
    key = feature_mapping_key(repo_id, control_mode)
    DATA_FEATURES_NAME_MAPPING[key] = dict(mapping)
    return key


def resolve_feature_mapping(repo_id: str, control_mode: str | None = None) -> dict[str, str]:
    """The precise ``"<repo_id>::<control_mode>"`` entry, else the plain ``repo_id`` entry; ``KeyError`` for neither."""
    for key in (feature_mapping_key(repo_id, control_mode), repo_id):
        if key in DATA_FEATURES_NAME_MAPPING:
            return DATA_FEATURES_NAME_MAPPING[key]
    raise KeyError(f"No feature mapping registered for repo_id={repo_id!r} (control_mode={control_mode!r}).")


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


def get_mapping(repo_id: str, features: dict[str, dict], override: dict[str, str] | None = None,
                control_mode: str | None = None) -> dict[str, str]:
    """The entry's own ``data_features_name_mapping`` when it has one, else the registered table (control-mode aware),
    else the conventional LeRobot names inferred from the feature dictionary."""
    if override:
        return dict(override)
    try:
        return dict(resolve_feature_mapping(repo_id, control_mode))
    except KeyError:
        return infer_mapping(features)
