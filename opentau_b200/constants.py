"""Names shared across the package: batch keys and checkpoint file layout.

Mirrors the reference's layout (OpenTau ``src/opentau/constants.py:39-49``,
``utils/train_utils.py:56-73``) so checkpoints are interchangeable.
"""

import os
from pathlib import Path

OBS_STATE = "state"
OBS_IMAGE_PREFIX = "camera"
ACTION = "actions"

CHECKPOINTS_DIR = "checkpoints"
LAST_CHECKPOINT_LINK = "last"
PRETRAINED_MODEL_DIR = "pretrained_model"
TRAINING_STATE_DIR = "training_state"
RNG_STATE = "rng_state.safetensors"
TRAINING_STEP = "training_step.json"
OPTIMIZER_STATE = "optimizer_state.safetensors"
OPTIMIZER_PARAM_GROUPS = "optimizer_param_groups.json"
SCHEDULER_STATE = "scheduler_state.json"
TRAIN_CONFIG_NAME = "train_config.json"
CONFIG_NAME = "config.json"
SAFETENSORS_SINGLE_FILE = "model.safetensors"
RUNNING_BEST_FILE = "running_best.json"

HF_OPENTAU_HOME = Path(os.environ.get("HF_OPENTAU_HOME", Path.home() / ".cache" / "opentau")).expanduser()
