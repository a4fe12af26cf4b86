"""Console entry points: ``opentau-train``, ``opentau-eval``, ``opentau-export``, ``opentau-dataset-viz``
(reference ``src/opentau/scripts/launch.py:30-99`` wraps ``accelerate launch``).

One process per GPU is started through ``torch.distributed.run`` on this node (rendezvous on 127.0.0.1).  The
``--accelerate-config <yaml>`` flag of the reference CLI is still accepted: its ``num_processes`` picks the rank
count and the file is forwarded to the script, which maps ``distributed_type`` onto the sharding strategy.
"""

from __future__ import annotations

import os
import subprocess
import sys


def _num_processes(argv: list[str]) -> tuple[int | None, list[str]]:
    n, rest = None, []
    it = iter(argv)
    for a in it:
        if a in ("--num-processes", "--num_processes", "--nproc-per-node"):
            n = int(next(it))
        elif a.startswith(("--num-processes=", "--num_processes=", "--nproc-per-node=")):
            n = int(a.split("=", 1)[1])
        else:
            rest.append(a)
    if n is None:
        for i, a in enumerate(rest):
            path = a.split("=", 1)[1] if a.startswith(("--accelerate-config=", "--accelerate_config=")) else (
                rest[i + 1] if a in ("--accelerate-config", "--accelerate_config") and i + 1 < len(rest) else None)
            if path and os.path.exists(path):
                import yaml
                with open(path) as f:
                    n = int((yaml.safe_load(f) or {}).get("num_processes", 0)) or None
    return n, rest


def build_command(module: str, argv: list[str]) -> tuple[list[str], dict[str, str]]:
    n, rest = _num_processes(argv)
    if n is None:
        try:
            import torch
            n = max(1, torch.cuda.device_count())
        except Exception:  # noqa: BLE001
            n = 1
    env = dict(os.environ)
    env.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    if n == 1:
        return [sys.executable, "-m", module, *rest], env
    port = env.get("MASTER_PORT", "29511")
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
            "--master-addr", "127.0.0.1", "--master-port", port, "-m", module, *rest], env


def launch(module: str, argv: list[str] | None = None) -> int:
    cmd, env = build_command(module, list(sys.argv[1:] if argv is None else argv))
    return subprocess.run(cmd, env=env).returncode


def train() -> None:
    sys.exit(launch("opentau_b200.scripts.train"))


def eval() -> None:  # noqa: A001 - name fixed by the console-script table
    sys.exit(launch("opentau_b200.scripts.eval"))


def export() -> None:
    sys.exit(launch("opentau_b200.scripts.export_to_onnx"))


def visualize() -> None:
    sys.exit(launch("opentau_b200.scripts.visualize_dataset"))
