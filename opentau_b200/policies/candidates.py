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
    """Learning-free critic: prefers the candidate closest to all the others, i.e. the chunk in the densest region
    of the sampled distribution.  A stand-in that makes best-of-N testable before a trained critic exists, not a
    quality model: on a multimodal task it prefers the more populated mode, not the better one.  Opt-in by name
    (``action_chunk_critic_path: "medoid"``).

    Raw action dims live on different scales (a gripper in [0, 1] against a joint in radians), so the distance is
    taken after dividing by the POLICY's per-dim scale for the sample's normalisation head, over the dims whose
    statistics show a spread and over the executed rows only.  The policy's un-normaliser is held by reference, not
    registered: this critic owns no tensors and its ``state_dict`` stays empty.  Without an un-normaliser (a bare
    ``MedoidCritic(max_action_dim=...)``) every dim counts with scale 1
    (reference ``src/opentau/policies/candidates.py:207-291``)."""

    def __init__(self, unnormalize: nn.Module | None = None, *, max_action_dim: int = 32):
        super().__init__()
        object.__setattr__(self, "_unnormalize", unnormalize)
        self.max_action_dim = int(max_action_dim)

    def score_chunks(self, batch, candidates: Tensor, *, row_mask: Tensor, dataset_index: Tensor) -> Tensor:
        del batch                                            # consensus is computed over the candidates alone
        B, N, T, D = candidates.shape
        if N < 3:
            raise ValueError(f"{type(self).__name__} needs n_candidates >= 3 to rank anything (got {N}): with two "
                             "candidates the single pairwise distance is shared, every score ties and selection "
                             "always falls back to candidate 0")
        row_mask = row_mask.to(device=candidates.device, dtype=torch.bool)
        if row_mask.ndim != 2:
            raise ValueError(f"row_mask must be (B, chunk) or (1, chunk); got {tuple(row_mask.shape)}")
        x = candidates.float()
        valid = row_mask.expand(B, T)[:, None, :, None]
        if self._unnormalize is not None:
            from .accel import action_dim_scale, resolve_action_dim_mask
            kw = dict(max_action_dim=max(self.max_action_dim, D), dataset_index=dataset_index)
            scale = action_dim_scale(self._unnormalize, **kw)[:, :D].to(x.device)
            keep = resolve_action_dim_mask(self._unnormalize, **kw)[:, :D].to(x.device)
            x = x / scale[:, None, None, :]
            valid = valid & keep[:, None, None, :]
        x = torch.where(valid, x, torch.zeros_like(x))
        flat = x.flatten(2)
        dist = torch.cdist(flat, flat)                       # (B, N, N); the zero self-distance adds nothing
        return -(dist.sum(-1) / (N - 1))


def collapse_candidates(t: Tensor, n: int) -> Tensor:
    """Inverse of :func:`expand_candidates`: ``(B * n, ...)`` -> ``(B, n, ...)``."""
    if t.shape[0] % n:
        raise ValueError(f"{t.shape[0]} rows do not split into groups of {n} candidates")
    return t.view(t.shape[0] // n, n, *t.shape[1:])


def pick(candidates: Tensor, index: Tensor) -> Tensor:
    """``candidates (B, N, ...)``, ``index (B,)`` -> ``(B, ...)``."""
    B = candidates.shape[0]
    return candidates[torch.arange(B, device=candidates.device), index]


def attach_critic(policy: nn.Module, critic: Any) -> None:
    """Binds ``critic`` to ``policy`` WITHOUT registering it: a plain attribute assignment of a module would put the
    critic's tensors into ``policy.state_dict()`` (and so into checkpoints) and its parameters into the optimizer.
    The price is that ``policy.to(...)`` does not move the critic; :func:`configure_candidates` places it
    (reference ``candidates.py:294-307``)."""
    object.__setattr__(policy, "_critic", critic)


def load_critic(path: str | None, *, policy: nn.Module) -> Any:
    """``action_chunk_critic_path`` -> a critic.  Only the built-in consensus selector exists; any other value names
    a learned critic and raises instead of silently selecting on nothing (reference ``candidates.py:310-323``)."""
    if path == MEDOID:
        return MedoidCritic(getattr(policy, "unnormalize_outputs", None), max_action_dim=policy.config.max_action_dim)
    raise NotImplementedError(f"action_chunk_critic_path={path!r} names a learned critic, which this build cannot "
                              f"load; only the built-in {MEDOID!r} selector is available")


def refuse_candidates(cfg: Any, *, reason: str) -> None:
    """For entry points that cannot honour best-of-N: raising beats silently ignoring ``n_candidates=4`` and letting
    the operator believe it is running (reference ``candidates.py:326-335``)."""
    requested = getattr(getattr(cfg, "policy", cfg), "n_candidates", 1) or 1
    if int(requested) > 1:
        raise ValueError(f"n_candidates={requested} is not supported here: {reason}")


def _smoke_critic(critic: Any, n: int, policy, device) -> None:
    """One call on dummy, DISTINCT candidates so that a critic returning the wrong shape fails at start-up, not on
    the first robot request (the protocol check sees only that the method exists)."""
    cfg = policy.config
    feat = getattr(cfg, "action_feature", None)
    dim = feat.shape[0] if feat is not None else cfg.max_action_dim
    probe = torch.arange(n, device=device, dtype=torch.float32).view(1, n, 1, 1).expand(1, n, cfg.chunk_size, dim)
    scores = critic.score_chunks({}, probe.contiguous(), row_mask=torch.ones(1, cfg.chunk_size, dtype=torch.bool,
                                                                           device=device),
                                 dataset_index=torch.zeros(1, dtype=torch.long, device=device))
    if not isinstance(scores, Tensor) or tuple(scores.shape) != (1, n):
        got = tuple(scores.shape) if isinstance(scores, Tensor) else type(scores).__name__
        raise TypeError(f"{type(critic).__name__}.score_chunks must return a (B, N) tensor; the probe with B=1, "
                        f"N={n} returned {got}")


def configure_candidates(policy, cfg: Any = None, critic: Any | None = None, *, device=None, dtype=None,
                         override: int | None = None) -> int:
    """The one knob every serving entry point uses to arm best-of-N; returns the resolved count.

    ``cfg`` is a pipeline / policy config (``n_candidates`` and ``action_chunk_critic_path`` are read from its
    ``policy`` section, or from itself) or, for direct use, the count as an integer.  ``override`` (an entry point's
    own flag) beats the config, and the precedence uses ``is None``, never truthiness: ``override=1`` deliberately
    DISABLES a config-enabled N.  ``critic`` may be an :class:`ActionChunkCritic`, the string ``"medoid"``, or
    ``None`` (then the config's path decides; with N > 1 and no path this raises).  N == 1 returns before any probe of
    the policy, so unarmed start-up works for every family; N > 1 on a family whose sampler does not read the
    setting is refused.  The critic is placed on ``device`` (default: the policy's), cast, put in eval mode and
    smoke-called here, so that a bad critic fails before warm-up (reference ``candidates.py:338-447``)."""
    if isinstance(cfg, int) and not isinstance(cfg, bool):
        requested, section = (cfg if override is None else override), policy.config
    else:
        section = getattr(cfg, "policy", cfg) if cfg is not None else policy.config
        requested = override if override is not None else getattr(section, "n_candidates", None)
    n = 1 if requested is None else int(requested)
    if n < 1:
        raise ValueError(f"n_candidates must be >= 1, got {n}")
    wired = hasattr(policy, "_n_candidates")
    if n == 1:
        if wired:                      # also in this case: a stale value from an earlier call must not survive
            policy._n_candidates = 1
            attach_critic(policy, None)
        return 1
    if not wired:
        kind = getattr(section, "type", type(policy).__name__)
        raise ValueError(f"n_candidates={n} was requested but policy type {kind!r} has no best-of-N sampler")
    if critic is None:
        critic = getattr(section, "action_chunk_critic_path", None)
        if critic is None:
            raise ValueError(f"n_candidates={n} needs a critic to choose between the candidates, but "
                             f"action_chunk_critic_path is unset; set it to {MEDOID!r} for the consensus selector")
    if isinstance(critic, str):
        critic = load_critic(critic, policy=policy)
    if not isinstance(critic, ActionChunkCritic):
        raise TypeError(f"{type(critic).__name__} does not satisfy the ActionChunkCritic protocol "
                        "(missing `score_chunks`)")
    if device is None:
        first = next(policy.parameters(), None)
        device = first.device if first is not None else torch.device("cpu")
    if isinstance(critic, nn.Module):
        critic.to(device=device, dtype=dtype) if dtype is not None else critic.to(device)
        critic.eval()
    _smoke_critic(critic, n, policy, device)
    attach_critic(policy, critic)
    policy._n_candidates = n
    logging.info("best-of-%d candidate sampling armed with %s", n, type(critic).__name__)
    return n
