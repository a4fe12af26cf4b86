"""Extract the Qwen3-VL "reasoner" weights from a Cosmos3 omni checkpoint into a standalone safetensors file that
the cosmos3 backbone loads (reference ``src/opentau/scripts/extract_cosmos3_reasoner.py``): keep the tensors under the
reasoner prefix, strip the prefix, and map them onto ``model.qwen3vl_with_expert.backbone.*``."""

from __future__ import annotations

import argparse
from pathlib import Path

DEFAULT_SRC_PREFIXES = ("reasoner.", "net.reasoner.", "model.reasoner.", "vlm.")
DST_PREFIX = "model.qwen3vl_with_expert.backbone."


def extract(state: dict, src_prefixes=DEFAULT_SRC_PREFIXES, dst_prefix: str = DST_PREFIX) -> dict:
    out = {}
    for k, v in state.items():
        for p in src_prefixes:
            if k.startswith(p):
                out[dst_prefix + k[len(p):]] = v
                break
    if not out:
        raise ValueError(f"no tensor starts with any of {list(src_prefixes)}")
    return out


def main(argv=None) -> None:
    from safetensors.torch import load_file, save_file
    ap = argparse.ArgumentParser()
    ap.add_argument("src", help="safetensors file or directory of shards")
    ap.add_argument("dst")
    ap.add_argument("--prefix", action="append", default=None)
    a = ap.parse_args(argv)
    files = sorted(Path(a.src).glob("*.safetensors")) if Path(a.src).is_dir() else [Path(a.src)]
    state = {}
    for f in files:
        state.update(load_file(str(f)))
    out = extract(state, tuple(a.prefix) if a.prefix else DEFAULT_SRC_PREFIXES)
    Path(a.dst).parent.mkdir(parents=True, exist_ok=True)
    save_file({k: v.contiguous() for k, v in out.items()}, a.dst)
    print(f"wrote {len(out)} tensors to {a.dst}")


if __name__ == "__main__":
    main()
