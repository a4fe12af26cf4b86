"""Helpers shared by the pi0.7 planner and controller."""

from __future__ import annotations

import torch
import torch.distributed as dist


def global_or_branch_decisions(presence_locals: tuple[bool, ...], any_locals: tuple[bool, ...],
                               field_names: tuple[str, ...], device: torch.device,
                               sync_across_ranks: bool = True) -> tuple[bool, ...]:
    """Makes the optional-prefix-block decisions identical on every rank with ONE int32 all-reduce.

    ``any_locals[i]`` (this rank's batch has at least one real entry for field i) is OR-reduced and returned:
    it selects Python branches that launch different numbers of kernels / collectives, so ranks must agree.
    ``presence_locals[i]`` (the field is a tensor rather than ``None`` on this rank) must be the same on all
    ranks; a disagreement is a programming error and raises on every rank
    (reference ``src/opentau/policies/pi07/low_level/modeling_pi07_low_level.py:93-191``).
    """
    n = len(field_names)
    if not (len(presence_locals) == len(any_locals) == n):
        raise ValueError("presence_locals, any_locals and field_names must have the same length")
    for a, p, name in zip(any_locals, presence_locals, field_names):
        if a and not p:
            raise ValueError(f"field {name!r} reports entries but is absent")
    if not (sync_across_ranks and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
        return tuple(bool(a) for a in any_locals)
    world = dist.get_world_size()
    dev = device if dist.get_backend() == "nccl" else torch.device("cpu")
    flags = torch.tensor([int(bool(a)) for a in any_locals] + [int(bool(p)) for p in presence_locals],
                         dtype=torch.int32, device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.SUM)
    vals = flags.tolist()
    bad = [field_names[i] for i in range(n) if vals[n + i] not in (0, world)]
    if bad:
        raise RuntimeError(f"ranks disagree on the presence of optional field(s) {bad}: every rank must pass the "
                           "same set of optional inputs (a tensor everywhere, or None everywhere)")
    return tuple(vals[i] > 0 for i in range(n))
