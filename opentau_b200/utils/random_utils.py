"""Seeding and RNG-state persistence.

Global RNGs are seeded with ``seed + process_index * 12345``; decisions that must agree across ranks use
explicit generators seeded from the config seed only (reference ``src/opentau/utils/random_utils.py:121-239``).
The RNG state of python / numpy / torch / cuda round-trips through ``rng_state.safetensors``.
"""

from __future__ import annotations

import random
from contextlib import contextmanager
from pathlib import Path
from typing import Any

import numpy as np
import torch

from ..constants import RNG_STATE

RANK_SEED_STRIDE = 12345


def set_seed(seed: int | None, process_index: int = 0) -> None:
    if seed is None:
        return
    s = int(seed) + int(process_index) * RANK_SEED_STRIDE
    random.seed(s)
    np.random.seed(s % (2**32))
    torch.manual_seed(s)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(s)


def serialize_python_rng_state() -> dict[str, torch.Tensor]:
    version, state, gauss = random.getstate()
    return {"py_rng_version": torch.tensor([version], dtype=torch.int64),
            "py_rng_state": torch.tensor(list(state), dtype=torch.int64)}


def deserialize_python_rng_state(d: dict[str, torch.Tensor]) -> None:
    random.setstate((int(d["py_rng_version"].item()), tuple(d["py_rng_state"].tolist()), None))


def serialize_numpy_rng_state() -> dict[str, torch.Tensor]:
    st = np.random.get_state()
    return {"np_rng_state_values": torch.tensor(st[1].astype(np.int64)),
            "np_rng_state_index": torch.tensor([st[2]], dtype=torch.int64),
            "np_rng_has_gauss": torch.tensor([st[3]], dtype=torch.int64),
            "np_rng_cached_gaussian": torch.tensor([st[4]], dtype=torch.float64)}


def deserialize_numpy_rng_state(d: dict[str, torch.Tensor]) -> None:
    np.random.set_state(("MT19937", d["np_rng_state_values"].numpy().astype(np.uint32),
                         int(d["np_rng_state_index"].item()), int(d["np_rng_has_gauss"].item()),
                         float(d["np_rng_cached_gaussian"].item())))


def serialize_torch_rng_state() -> dict[str, torch.Tensor]:
    out = {"torch_rng_state": torch.get_rng_state()}
    if torch.cuda.is_available():
        out["torch_cuda_rng_state"] = torch.cuda.get_rng_state()
    return out


def deserialize_torch_rng_state(d: dict[str, torch.Tensor]) -> None:
    torch.set_rng_state(d["torch_rng_state"].to(torch.uint8).cpu())
    if torch.cuda.is_available() and "torch_cuda_rng_state" in d:
        torch.cuda.set_rng_state(d["torch_cuda_rng_state"].to(torch.uint8).cpu())


def get_rng_state() -> dict:
    """The live states of ``random``, ``numpy.random`` and ``torch`` (and the current CUDA device's generator) as
    plain Python objects: for bracketing a block in memory (:func:`seeded_context`), not for files
    (reference ``src/opentau/utils/random_utils.py:176-203``)."""
    import random
    state = {"random_state": random.getstate(), "numpy_random_state": np.random.get_state(),
             "torch_random_state": torch.random.get_rng_state()}
    if torch.cuda.is_available():
        state["torch_cuda_random_state"] = torch.cuda.random.get_rng_state()
    return state


def set_rng_state(state: dict) -> None:
    import random
    random.setstate(state["random_state"])
    np.random.set_state(state["numpy_random_state"])
    torch.random.set_rng_state(state["torch_random_state"])
    if torch.cuda.is_available() and "torch_cuda_random_state" in state:
        torch.cuda.random.set_rng_state(state["torch_cuda_random_state"])


def serialize_rng_state() -> dict[str, torch.Tensor]:
    return {**serialize_python_rng_state(), **serialize_numpy_rng_state(), **serialize_torch_rng_state()}


def deserialize_rng_state(d: dict[str, torch.Tensor]) -> None:
    deserialize_python_rng_state(d)
    deserialize_numpy_rng_state(d)
    deserialize_torch_rng_state(d)


def rng_state_file(save_dir: Path, rank: int | None = None) -> Path:
    """``rng_state.safetensors`` (single process) or ``rng_state_rank<r>.safetensors`` (one per rank: every rank
    draws its own flow-matching noise / time / augmentation stream, so every rank saves and restores its own;
    the reference keeps one ``random_states_<i>.pkl`` per process, ``utils/train_utils.py:115-132``)."""
    if rank is None:
        return Path(save_dir) / RNG_STATE
    stem, ext = RNG_STATE.rsplit(".", 1)
    return Path(save_dir) / f"{stem}_rank{rank}.{ext}"


def save_rng_state(save_dir: Path, rank: int | None = None) -> None:
    from safetensors.torch import save_file
    save_dir.mkdir(parents=True, exist_ok=True)
    save_file({k: v.contiguous() for k, v in serialize_rng_state().items()}, str(rng_state_file(save_dir, rank)))


def load_rng_state(save_dir: Path, rank: int | None = None) -> None:
    """Restores this rank's stream; raises FileNotFoundError when the checkpoint holds none for it."""
    from safetensors.torch import load_file
    f = rng_state_file(save_dir, rank)
    if not f.exists() and rank == 0 and (Path(save_dir) / RNG_STATE).exists():
        f = Path(save_dir) / RNG_STATE          # checkpoints written before the per-rank files existed
    if not f.exists():
        raise FileNotFoundError(str(f))
    deserialize_rng_state(load_file(str(f)))


@contextmanager
def seeded_context(seed: int | None):
    """Runs a block under a temporary seed and restores the previous RNG state afterwards."""
    state = serialize_rng_state()
    set_seed(seed)
    try:
        yield
    finally:
        deserialize_rng_state(state)


def rank_generator(seed: int, rank_independent: bool = True, process_index: int = 0) -> torch.Generator:
    g = torch.Generator()
    g.manual_seed(int(seed) + (0 if rank_independent else process_index * RANK_SEED_STRIDE))
    return g
