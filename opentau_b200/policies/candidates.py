"""Best-of-N action chunks: one prefix pass, N noise draws through the expert, a critic keeps one.

The prefix KV cache is never written during denoising, so it is widened (as a view) across candidates and
the extra cost is only a wider expert batch.  Off unless an entry point arms it with
:func:`configure_candidates` (reference ``src/opentau/policies/candidates.py:94-475``).
"""

from __future__ import annotations

import logging
import math
from typing import Any, Protocol, runtime_checkable

import torch
from torch import Tensor, nn

MEDOID = "medoid"


@runtime_checkable
class ActionChunkCritic(Protocol):
    def score_chunks(self, batch: dict[str, Tensor], candidates: Tensor, *, row_mask: Tensor,
                     dataset_index: Tensor) -> Tensor:
        """``candidates (B, N, chunk, dim)`` in raw units -> scores ``(B, N)``, higher is better."""
        ...


def expand_candidates(t: Tensor | None, n: int) -> Tensor | None:
    """Repeats batch rows ``n`` times (row i -> rows i*n .. i*n+n-1)."""
    if t is None or n == 1:
        return t
    return t.repeat_interleave(n, dim=0)


def expand_kv_cache(cache, n: int):
    """Widens a prefix cache to ``B * n`` rows without copying when ``B == 1``."""
    return cache.expand_batch(n) if n > 1 else cache


def select_candidate(scores: Tensor) -> Tensor:
    """Argmax over finite scores per row; a row with no finite score falls back to candidate 0.

    Total by design (never raises: a data-dependent raise on one rank would leave its peers blocked in
    the next collective); NaN never wins; ties go to the lowest index, so a degenerate critic reduces to
    the single-sample behaviour."""
    finite = torch.isfinite(scores)
    masked = torch.where(finite, scores.float(), torch.full_like(scores, float("-inf"), dtype=torch.float32))
    all_bad = ~finite.any(dim=1)
    safe = torch.where(all_bad[:, None], torch.zeros_like(masked), masked)
    picked = torch.argmax(safe, dim=1)
    return torch.where(all_bad, torch.zeros_like(picked), picked)


_WARNED = False


def warn_if_no_candidate_scored(score_rows: list[list[float]]) -> None:
    global _WARNED
    if _WARNED:
        return
    bad = [i for i, row in enumerate(score_rows) if not any(math.isfinite(v) for v in row)]
    if bad:
        _WARNED = True
        logging.warning("action-chunk critic returned no finite score for batch row(s) %s; they fell back to "
                        "candidate 0 (logged once per process)", bad)


class MedoidCritic(nn.Module):
    """Learning-free critic: prefers the candidate closest (on executed rows, real dims, per-dim scaled) to
    all the others — the chunk in the densest region of the sampled distribution."""

    def __init__(self, dim_scale: Tensor | None = None, max_action_dim: int = 32):
        super().__init__()
        self.max_action_dim = max_action_dim
        self.register_buffer("dim_scale", dim_scale if dim_scale is not None else torch.ones(max_action_dim),
                             persistent=False)

    def score_chunks(self, batch, candidates: Tensor, *, row_mask: Tensor, dataset_index: Tensor) -> Tensor:
        B, N, T, D = candidates.shape
        if N == 1:
            return torch.zeros(B, 1, device=candidates.device)
        if N == 2:
            logging.debug("with two candidates the single pairwise distance is shared: every score ties")
        x = candidates.float() / self.dim_scale[:D].to(candidates.device).clamp_min(1e-6)
        x = x * row_mask.to(x.dtype).expand(B, T)[:, None, :, None]
        flat = x.flatten(2)
        dist = torch.cdist(flat, flat)                      # (B, N, N)
        return -(dist.sum(-1) / (N - 1))


def pick(candidates: Tensor, index: Tensor) -> Tensor:
    """``candidates (B, N, ...)``, ``index (B,)`` -> ``(B, ...)``."""
    B = candidates.shape[0]
    return candidates[torch.arange(B, device=candidates.device), index]


def configure_candidates(policy, n_candidates: int | None, critic: Any | None = None) -> None:
    """The only writer of a policy's best-of-N setting.  ``critic`` may be an object implementing
    :class:`ActionChunkCritic`, the string ``"medoid"``, or ``None`` (with N > 1 this raises)."""
    n = int(n_candidates or 1)
    if n < 1:
        raise ValueError("n_candidates must be >= 1")
    if n > 1:
        if critic is None:
            critic = getattr(policy.config, "action_chunk_critic_path", None)
        if critic == MEDOID:
            critic = MedoidCritic(max_action_dim=policy.config.max_action_dim)
        if critic is None or isinstance(critic, str) or not isinstance(critic, ActionChunkCritic):
            raise ValueError("best-of-N needs a critic: pass one, or set action_chunk_critic_path='medoid'")
    policy._n_candidates = n
    policy._critic = critic if n > 1 else None
