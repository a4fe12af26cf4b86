"""Synthetic batches in the standard data format (random images, prompts, states, action chunks).

Used by benchmarks, profilers and tests: uniform-random uint8-like images in [0,1], uniform prompt
token ids, ``N(0,1)`` state and actions, uniform FAST-style action tokens — the shapes named by the
benchmark configurations.  Keys follow the batch schema of the reference
(OpenTau ``src/opentau/datasets/lerobot_dataset.py:975-1072``); pre-tokenised ``lang_tokens`` and
``discrete_actions`` replace the CPU tokenisers so the data path has no per-step host work.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import Tensor


@dataclass
class SyntheticSpec:
    batch_size: int = 4
    num_cams: int = 1
    resolution: tuple[int, int] = (224, 224)
    prompt_len: int = 16
    vocab_size: int = 1024
    state_dim: int = 8
    action_dim: int = 8
    max_state_dim: int = 32
    max_action_dim: int = 32
    chunk_size: int = 10
    discrete_action_len: int = 8
    discrete_action_vocab: int = 256
    image_dtype: torch.dtype = torch.float32


def make_synthetic_batch(spec: SyntheticSpec, device="cpu", seed: int = 0, pinned: bool = False) -> dict[str, Tensor]:
    g = torch.Generator().manual_seed(seed)
    B = spec.batch_size
    out: dict[str, Tensor] = {}
    for c in range(spec.num_cams):
        img = torch.randint(0, 256, (B, 3, *spec.resolution), generator=g, dtype=torch.uint8)
        out[f"camera{c}"] = (img.to(torch.float32) / 255.0).to(spec.image_dtype)
    state = torch.zeros(B, spec.max_state_dim)
    state[:, :spec.state_dim] = torch.randn(B, spec.state_dim, generator=g)
    actions = torch.zeros(B, spec.chunk_size, spec.max_action_dim)
    actions[:, :, :spec.action_dim] = torch.randn(B, spec.chunk_size, spec.action_dim, generator=g)
    out["state"] = state
    out["actions"] = actions
    out["lang_tokens"] = torch.randint(3, spec.vocab_size, (B, spec.prompt_len), generator=g)
    out["lang_masks"] = torch.ones(B, spec.prompt_len, dtype=torch.bool)
    out["discrete_actions"] = torch.randint(1, spec.discrete_action_vocab, (B, spec.discrete_action_len), generator=g)
    out["discrete_action_masks"] = torch.ones(B, spec.discrete_action_len, dtype=torch.bool)
    out["img_is_pad"] = torch.zeros(B, spec.num_cams, dtype=torch.bool)
    out["action_is_pad"] = torch.zeros(B, spec.chunk_size, dtype=torch.bool)
    out["real_action_dim"] = torch.full((B,), spec.action_dim, dtype=torch.long)
    out["dataset_index"] = torch.zeros(B, dtype=torch.long)
    if pinned and torch.cuda.is_available():
        out = {k: v.pin_memory() for k, v in out.items()}
    if str(device) != "cpu":
        out = {k: v.to(device, non_blocking=True) for k, v in out.items()}
    return out


def identity_stats(max_state_dim: int = 32, max_action_dim: int = 32) -> dict:
    """Statistics under which normalisation is (nearly) the identity: mean 0/std 1, range [-1, 1]."""
    import numpy as np
    return {
        "state": {"min": -np.ones(max_state_dim, np.float32), "max": np.ones(max_state_dim, np.float32),
                  "mean": np.zeros(max_state_dim, np.float32), "std": np.ones(max_state_dim, np.float32)},
        "actions": {"min": -np.ones(max_action_dim, np.float32), "max": np.ones(max_action_dim, np.float32),
                    "mean": np.zeros(max_action_dim, np.float32), "std": np.ones(max_action_dim, np.float32)},
    }
