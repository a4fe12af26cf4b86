"""Stable names for serial adapters and cameras (reference ``src/opentau/scripts/so101/device_paths.py:17-85``).

``/dev/ttyACM<n>`` and ``/dev/video<n>`` are numbered in enumeration order and move between boots and replugs.  udev
keeps aliases that do not: ``/dev/serial/by-id/`` (keyed by the adapter's USB serial number: it follows an arm to
whichever socket it is plugged into, the right key for a motor bus) and ``/dev/v4l/by-path/`` (keyed by the USB
topology: the right key for cameras, because identical camera models often share one serial number and their
``by-id`` links collide).  Without udev (macOS, Windows, most containers) every helper answers "no stable name".
"""

from __future__ import annotations

import os
from pathlib import Path

SERIAL_BY_ID_DIR = Path("/dev/serial/by-id")
VIDEO_BY_PATH_DIR = Path("/dev/v4l/by-path")


def stable_link_map(link_dir: str | Path) -> dict[str, str]:
    """``{real device node: alias}`` for the symlinks in ``link_dir``.  One node can have several aliases (a V4L device
    usually has a ``-usb-`` and a ``-usbv2-`` link); names are visited in sorted order and the first wins, so the
    answer is the same on every run.  A missing or unreadable directory gives ``{}``."""
    try:
        links = sorted(Path(link_dir).iterdir())
    except OSError:
        return {}
    out: dict[str, str] = {}
    for link in links:
        try:
            out.setdefault(os.path.realpath(link), str(link))
        except OSError:
            continue
    return out


def _stable(device, link_dir: Path) -> str | None:
    if not isinstance(device, str):          # bare camera indices (no udev) have no alias
        return None
    try:
        return stable_link_map(link_dir).get(os.path.realpath(device))
    except OSError:
        return None


def stable_serial_path(device, link_dir: Path | None = None) -> str | None:
    """``/dev/ttyACM0`` -> ``/dev/serial/by-id/usb-...`` or None."""
    return _stable(device, link_dir or SERIAL_BY_ID_DIR)


def stable_video_path(device, link_dir: Path | None = None) -> str | None:
    """``/dev/video0`` -> ``/dev/v4l/by-path/pci-...`` or None."""
    return _stable(device, link_dir or VIDEO_BY_PATH_DIR)
