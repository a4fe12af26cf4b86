"""Optional-dependency probes (reference ``src/opentau/utils/import_utils.py:20-79``)."""

from __future__ import annotations

import importlib
import importlib.metadata
import logging


def is_package_available(pkg_name: str, return_version: bool = False):
    exists = importlib.util.find_spec(pkg_name) is not None
    version = "N/A"
    if exists:
        try:
            version = importlib.metadata.version(pkg_name)
        except importlib.metadata.PackageNotFoundError:
            try:
                version = getattr(importlib.import_module(pkg_name), "__version__", "N/A")
            except ImportError:
                exists = False
        logging.debug("Detected %s version: %s", pkg_name, version)
    return (exists, version) if return_version else exists


_wandb_available = is_package_available("wandb")
_grpc_available = is_package_available("grpc")
_cv2_available = is_package_available("cv2")
_onnx_available = is_package_available("onnx")
_gym_available = is_package_available("gymnasium")
