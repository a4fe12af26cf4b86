"""Fetch simulator assets: the LIBERO benchmark files and the RoboCasa kitchen assets.

The reference has one script per simulator (``src/opentau/scripts/download_libero_benchmarks.py``,
``download_robocasa_assets.py``); both call the simulator package's own downloader after checking that the package is
importable.  Here they are one module with two entry points.  Without the simulator package, or without network access,
the call explains what is missing instead of failing half-way.

    python -m opentau_b200.scripts.download_assets libero [--datasets libero_10 ...]
    python -m opentau_b200.scripts.download_assets robocasa
"""

from __future__ import annotations

import argparse
import importlib
import importlib.util
import socket


def online(host: str = "huggingface.co", timeout: float = 2.0) -> bool:
    try:
        socket.create_connection((host, 443), timeout=timeout).close()
        return True
    except OSError:
        return False


def download_libero(datasets: list[str] | None = None) -> int:
    if importlib.util.find_spec("libero") is None:
        print("the `libero` package is not installed: nothing to download into")
        return 2
    if not online():
        print("no network access: LIBERO benchmark files cannot be fetched from this machine")
        return 3
    mod = importlib.import_module("libero.libero.utils.download_utils")     # pragma: no cover - needs the simulator
    for name in datasets or ["libero_spatial", "libero_object", "libero_goal", "libero_10"]:
        mod.libero_dataset_download(datasets=name, use_huggingface=True)
    return 0


def download_robocasa() -> int:
    if importlib.util.find_spec("robocasa") is None:
        print("the `robocasa` package is not installed: nothing to download into")
        return 2
    if not online("utexas.box.com"):
        print("no network access: RoboCasa kitchen assets cannot be fetched from this machine")
        return 3
    mod = importlib.import_module("robocasa.scripts.download_kitchen_assets")  # pragma: no cover - needs the simulator
    mod.main()
    return 0


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["libero", "robocasa"])
    ap.add_argument("--datasets", nargs="*", default=None)
    a = ap.parse_args(argv)
    return download_libero(a.datasets) if a.what == "libero" else download_robocasa()


if __name__ == "__main__":
    raise SystemExit(main())
