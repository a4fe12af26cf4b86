"""Checkpoint layout, pruning, resume and the running-best tracker.

Directory layout (same as the reference, OpenTau ``src/opentau/utils/train_utils.py:56-489``):

    <output_dir>/checkpoints/<step, zero-padded to >= 6 digits>/
        model.safetensors, config.json          policy weights + policy config
        train_config.json                       the full pipeline config
        training_step.json                      {"step": N}
        rng_state_rank<r>.safetensors           python / numpy / torch / cuda RNG of rank r (one file per rank)
        optimizer_rank<r>.safetensors           this rank's shard of Adam moments (+ fp32 masters)
        flat_layout.json                        parameter name / shape / offset inside the flat groups
        random_states_<r>.marker                one per rank: the completeness tripwire counts them
    <output_dir>/checkpoints/last -> <step>     symlink
    <output_dir>/checkpoints/running_best.json  RunningBestTracker state
"""

from __future__ import annotations

import json
import logging
import os
import shutil
from pathlib import Path
from typing import Any

import torch

from ..constants import (CHECKPOINTS_DIR, LAST_CHECKPOINT_LINK, RUNNING_BEST_FILE, TRAINING_STEP)
from .random_utils import load_rng_state, save_rng_state, set_seed


def get_step_identifier(step: int, total_steps: int) -> str:
    width = max(6, len(str(total_steps)))
    return f"{step:0{width}d}"


def get_step_checkpoint_dir(output_dir: Path | str, total_steps: int, step: int) -> Path:
    return Path(output_dir) / CHECKPOINTS_DIR / get_step_identifier(step, total_steps)


def save_training_step(step: int, save_dir: Path) -> None:
    save_dir.mkdir(parents=True, exist_ok=True)
    with open(save_dir / TRAINING_STEP, "w") as f:
        json.dump({"step": step}, f)


def load_training_step(save_dir: Path) -> int:
    with open(save_dir / TRAINING_STEP) as f:
        return int(json.load(f)["step"])


def update_last_checkpoint(checkpoint_dir: Path) -> Path:
    link = checkpoint_dir.parent / LAST_CHECKPOINT_LINK
    if link.is_symlink() or link.exists():
        link.unlink()
    link.symlink_to(checkpoint_dir.name)
    return link


def save_checkpoint(checkpoint_dir: Path, step: int, cfg, policy, engine=None, rank: int = 0,
                    is_main: bool = True) -> None:
    """Rank 0 writes the policy / configs / step; every rank writes its RNG state, its optimizer shard and, last,
    its marker.  Every rank must call this (no rank may decide on its own from the directory's existence)."""
    from safetensors.torch import save_file
    checkpoint_dir.mkdir(parents=True, exist_ok=True)
    # a parameter-sharded engine holds 1 / W of every weight: all ranks gather (a collective), rank 0 writes
    import contextlib
    with (engine.full_params() if hasattr(engine, "full_params") else contextlib.nullcontext()):
        if is_main:
            policy.save_pretrained(checkpoint_dir)
    if is_main:
        cfg.save_pretrained(checkpoint_dir)
        save_training_step(step, checkpoint_dir)
        (checkpoint_dir / "world_size.json").write_text(json.dumps({"world_size": getattr(engine, "world", 1)}))
    save_rng_state(checkpoint_dir, rank)
    if engine is not None and is_main:
        with open(checkpoint_dir / "flat_layout.json", "w") as f:
            json.dump(engine.store.layout(), f)
    if engine is not None:
        sd = engine.state_dict()
        tensors = {k: v.detach().cpu().contiguous() for k, v in sd.items() if isinstance(v, torch.Tensor)}
        meta = {k: str(v) for k, v in sd.items() if not isinstance(v, torch.Tensor)}
        save_file(tensors, str(checkpoint_dir / f"optimizer_rank{rank}.safetensors"), metadata=meta)
    (checkpoint_dir / f"random_states_{rank}.marker").write_text(str(step))


def saved_world_size(checkpoint_dir: Path) -> int:
    """World size the checkpoint was written with (1 for checkpoints that predate the record)."""
    f = Path(checkpoint_dir) / "world_size.json"
    if f.exists():
        return int(json.loads(f.read_text())["world_size"])
    return max(1, len(list(Path(checkpoint_dir).glob("optimizer_rank*.safetensors"))))


def checkpoint_is_complete(checkpoint_dir: Path, world_size: int | None = None) -> bool:
    """Tripwire for interrupted saves: one marker per rank of the SAVING job must exist."""
    if world_size is None:
        world_size = saved_world_size(checkpoint_dir)
    return len(list(checkpoint_dir.glob("random_states_*.marker"))) >= world_size


def load_training_state(checkpoint_dir: Path, engine=None, rank: int = 0, world_size: int = 1,
                        seed: int | None = None) -> int:
    """Restores step, RNG and this rank's optimizer shard.  When the world size changed since the save the
    Adam moments cannot be re-sharded in place: masters are rebuilt from the live bf16 weights, moments
    restart at zero, and ranks beyond the saved world are reseeded deterministically."""
    from safetensors import safe_open
    step = load_training_step(checkpoint_dir)
    try:
        load_rng_state(checkpoint_dir, rank)
    except FileNotFoundError:
        # a rank the checkpoint never had (world grew) or a checkpoint without RNG files: a fresh, rank-specific,
        # step-specific stream -- never another rank's
        logging.warning("no RNG state for rank %d in %s; reseeding from (seed, step, rank)", rank, checkpoint_dir)
        if seed is not None:
            set_seed(seed + step, rank)
    if engine is not None:
        f = checkpoint_dir / f"optimizer_rank{rank}.safetensors"
        saved_world = len(list(checkpoint_dir.glob("optimizer_rank*.safetensors")))
        if f.exists() and saved_world == world_size:
            sd: dict[str, Any] = {}
            with safe_open(str(f), framework="pt") as g:
                for k in g.keys():
                    sd[k] = g.get_tensor(k)
                for k, v in (g.metadata() or {}).items():
                    sd[k] = int(v) if v.lstrip("-").isdigit() else v
            sd["step"] = step
            engine.load_state_dict(sd)
        else:
            logging.warning("optimizer shards were saved for world size %d, now %d: rebuilding fp32 masters from "
                            "the live weights and restarting Adam moments", saved_world, world_size)
            engine.step_count = step
            engine.rebuild_masters_from_live()
    return step


def prune_checkpoints(output_dir: Path, keep: set[str]) -> None:
    root = Path(output_dir) / CHECKPOINTS_DIR
    if not root.is_dir():
        return
    for d in root.iterdir():
        if d.is_dir() and not d.is_symlink() and d.name not in keep:
            shutil.rmtree(d, ignore_errors=True)


class RunningBestTracker:
    """Keeps the ``count`` best checkpoints by a metric (lower is better for losses, higher for success)."""

    def __init__(self, output_dir: Path | str, count: int, metric: str = "auto", higher_is_better: bool = False):
        self.path = Path(output_dir) / CHECKPOINTS_DIR / RUNNING_BEST_FILE
        self.count, self.metric, self.higher_is_better = count, metric, higher_is_better
        self.entries: list[dict[str, Any]] = []
        if self.path.exists():
            self.entries = json.loads(self.path.read_text()).get("entries", [])

    def would_keep(self, value: float) -> bool:
        if self.count <= 0:
            return False
        if len(self.entries) < self.count:
            return True
        worst = self.entries[-1]["value"]
        return value > worst if self.higher_is_better else value < worst

    def update(self, step_id: str, value: float) -> list[str]:
        """Registers a checkpoint; returns the step ids that fell out of the top-``count``."""
        self.entries.append({"step": step_id, "value": float(value)})
        self.entries.sort(key=lambda e: e["value"], reverse=self.higher_is_better)
        dropped = [e["step"] for e in self.entries[self.count:]]
        self.entries = self.entries[: self.count]
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self.path.write_text(json.dumps({"metric": self.metric, "higher_is_better": self.higher_is_better,
                                         "entries": self.entries}, indent=2))
        return dropped

    @property
    def kept(self) -> set[str]:
        return {e["step"] for e in self.entries}
