"""ctypes loader for the in-tree native libraries (``_native/libotb_*.so``).

Loading is lazy and strict: asking for a library that is not built raises with the build command.
Set ``OPENTAU_B200_AUTOBUILD=1`` to compile on first use (needs nvcc).
"""

from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

from . import build as _build

_lock = threading.Lock()
_libs: dict[str, ctypes.CDLL] = {}


def load(name: str) -> ctypes.CDLL:
    with _lock:
        if name in _libs:
            return _libs[name]
        path = _build.lib_path(name)
        if not path.exists():
            if os.environ.get("OPENTAU_B200_AUTOBUILD", "0") == "1":
                _build.build_one(name)
            else:
                raise RuntimeError(
                    f"native library {path.name} is not built; run `python -m opentau_b200.ops.build` "
                    "(or __graft_entry__.build()) first")
        lib = ctypes.CDLL(str(path))
        _libs[name] = lib
        return lib


def loaded_libraries() -> list[str]:
    return [str(_build.lib_path(n)) for n in _libs]
