"""``pytorch_model.bin`` -> ``model.safetensors`` (reference ``src/opentau/scripts/bin_to_safetensors.py:30-116``);
tensors that share storage are cloned, normalisation buffers are kept."""

from __future__ import annotations

import argparse
from pathlib import Path

import torch


def convert(src: str | Path, dst: str | Path) -> int:
    from safetensors.torch import save_file
    sd = torch.load(str(src), map_location="cpu", weights_only=True)
    if "state_dict" in sd and isinstance(sd["state_dict"], dict):
        sd = sd["state_dict"]
    seen: dict[int, str] = {}
    out = {}
    for k, v in sd.items():
        if not isinstance(v, torch.Tensor):
            continue
        k = k[7:] if k.startswith("module.") else k
        ptr = v.untyped_storage().data_ptr()
        out[k] = v.clone().contiguous() if ptr in seen else v.contiguous()
        seen[ptr] = k
    Path(dst).parent.mkdir(parents=True, exist_ok=True)
    save_file(out, str(dst))
    return len(out)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("src")
    ap.add_argument("dst")
    a = ap.parse_args()
    print(f"wrote {convert(a.src, a.dst)} tensors to {a.dst}")


if __name__ == "__main__":
    main()
