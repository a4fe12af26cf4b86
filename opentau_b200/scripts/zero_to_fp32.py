"""Merge the per-rank optimizer shards of a checkpoint into one full-precision state dict.

The reference ships DeepSpeed's ``zero_to_fp32.py`` for its ZeRO checkpoints (``src/opentau/scripts/zero_to_fp32.py``,
used by ``convert_checkpoint.sh``).  Here every rank saves its slices ``[lo, hi)`` (one per gradient bucket) of each flat parameter group as
``optimizer_rank<r>.safetensors`` (fp32 masters and Adam moments) and rank 0 saves ``flat_layout.json`` (parameter name,
shape and offset inside the flat groups), so the consolidation is a concatenation followed by slicing:

    python -m opentau_b200.scripts.zero_to_fp32 <checkpoint_dir> <output.safetensors> [--moments]

The output holds the fp32 master of every trainable parameter under its ``state_dict`` name (frozen parameters and
buffers are taken from ``model.safetensors`` unchanged); ``--moments`` adds ``<name>.exp_avg`` / ``<name>.exp_avg_sq``.
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch


def _load(path: Path) -> tuple[dict[str, torch.Tensor], dict[str, str]]:
    from safetensors import safe_open
    with safe_open(str(path), framework="pt") as f:
        return {k: f.get_tensor(k) for k in f.keys()}, dict(f.metadata() or {})


def merge_flat(checkpoint_dir: str | Path, what: str = "master") -> list[torch.Tensor | None]:
    """One full flat fp32 tensor per group (None when no rank stored ``what`` for it)."""
    ckpt = Path(checkpoint_dir)
    layout = json.loads((ckpt / "flat_layout.json").read_text())
    files = sorted(ckpt.glob("optimizer_rank*.safetensors"), key=lambda p: int(p.stem.removeprefix("optimizer_rank")))
    if not files:
        raise FileNotFoundError(f"no optimizer_rank*.safetensors in {ckpt}")
    shards = [_load(f) for f in files]
    out: list[torch.Tensor | None] = []
    for gi, g in enumerate(layout):
        key = f"group{gi}.{what}"
        if not any(key in t for t, _ in shards):
            out.append(None)
            continue
        flat = torch.zeros(g["numel"], dtype=torch.float32)
        covered = 0
        for tensors, meta in shards:
            if f"group{gi}.slices" in tensors:           # one [lo, hi) per gradient bucket, stored back to back
                slices = tensors[f"group{gi}.slices"].reshape(-1, 2).tolist()
            else:                                        # older checkpoints: one contiguous range per rank
                slices = [[int(meta[f"group{gi}.lo"]), int(meta[f"group{gi}.hi"])]]
            off = 0
            for lo, hi in slices:
                flat[lo:hi] = tensors[key][off:off + hi - lo].float()
                off += hi - lo
                covered += hi - lo
        if covered < g["numel"]:
            raise ValueError(f"group {gi}: shards cover {covered} of {g['numel']} elements (a rank file is missing)")
        out.append(flat)
    return out


def consolidate(checkpoint_dir: str | Path, moments: bool = False) -> dict[str, torch.Tensor]:
    ckpt = Path(checkpoint_dir)
    layout = json.loads((ckpt / "flat_layout.json").read_text())
    state, _ = _load(ckpt / "model.safetensors") if (ckpt / "model.safetensors").exists() else ({}, {})
    state = {k: v for k, v in state.items()}
    names = {"master": "", "m": ".exp_avg", "v": ".exp_avg_sq"}
    for what in (("master", "m", "v") if moments else ("master",)):
        for g, flat in zip(layout, merge_flat(ckpt, what)):
            if flat is None:
                continue
            for p in g["params"]:
                n = 1
                for d in p["shape"]:
                    n *= d
                state[p["name"] + names[what]] = flat[p["offset"]:p["offset"] + n].view(p["shape"]).clone()
    return state


def main(argv: list[str] | None = None) -> None:
    from safetensors.torch import save_file
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("checkpoint_dir")
    ap.add_argument("output")
    ap.add_argument("--moments", action="store_true")
    a = ap.parse_args(argv)
    state = consolidate(a.checkpoint_dir, a.moments)
    save_file({k: v.contiguous() for k, v in state.items()}, a.output)
    print(f"{len(state)} tensors -> {a.output}")


if __name__ == "__main__":
    main()
