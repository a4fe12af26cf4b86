"""``python -m opentau_b200.scripts.display_sys_info [--json]``: the facts a bug report needs (reference
``src/opentau/scripts/display_sys_info.py``): interpreter, platform, torch / CUDA / cuDNN / NCCL versions, every
visible GPU with memory and compute capability, the optional packages this framework can use, and which of its
native extensions are built."""

from __future__ import annotations

import argparse
import importlib
import json
import platform

import torch


def collect() -> dict:
    info: dict = {"python": platform.python_version(), "platform": platform.platform(), "torch": torch.__version__,
                  "cuda_runtime": str(torch.version.cuda), "cuda_available": torch.cuda.is_available(),
                  "cudnn": str(torch.backends.cudnn.version()) if torch.backends.cudnn.is_available() else None}
    try:
        info["nccl"] = ".".join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else None
    except Exception:                                            # builds without NCCL
        info["nccl"] = None
    gpus = []
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        gpus.append({"index": i, "name": p.name, "memory_gib": round(p.total_memory / 2**30, 1),
                     "capability": f"{p.major}.{p.minor}", "sms": p.multi_processor_count})
    info["gpus"] = gpus
    pkgs = {}
    for name in ("transformers", "safetensors", "numpy", "pyarrow", "cv2", "onnx", "onnxruntime", "grpc", "wandb"):
        try:
            pkgs[name] = getattr(importlib.import_module(name), "__version__", "present")
        except Exception:
            pkgs[name] = None
    info["packages"] = pkgs
    from ..ops import build
    info["native_extensions"] = {n: build.lib_path(n).exists() for n in build.SOURCES}
    return info


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    info = collect()
    if a.json:
        print(json.dumps(info, indent=2))
    else:
        for k, v in info.items():
            if isinstance(v, dict):
                print(f"{k}:")
                for kk, vv in v.items():
                    print(f"  {kk:24s} {vv}")
            elif isinstance(v, list):
                print(f"{k}:")
                for g in v:
                    print("  " + ", ".join(f"{a_}={b_}" for a_, b_ in g.items()))
            else:
                print(f"{k:18s} {v}")
    return info


if __name__ == "__main__":
    main()
