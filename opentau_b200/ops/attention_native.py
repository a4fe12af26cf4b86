"""ctypes launcher of the tcgen05 block-causal attention kernels."""

from __future__ import annotations

import os

from torch import Tensor


def available() -> bool:
    from . import build
    return build.lib_path("attention_tcgen05").exists() and os.environ.get("OPENTAU_B200_DENSE_ATTN", "0") != "1"


def supported(q: Tensor, k: Tensor, v: Tensor) -> bool:
    return False


def supported_bwd(q: Tensor, k: Tensor, v: Tensor) -> bool:
    return False
