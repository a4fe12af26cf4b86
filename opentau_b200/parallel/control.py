"""Control-plane collectives on ``torch.distributed`` (NCCL or gloo): barriers, scalar metric gathers,
object broadcast/gather, OR-reduced branch decisions.  World size 1 degrades to identities.

These replace the ``accelerate`` utility calls of the reference training loop
(OpenTau ``src/opentau/scripts/train.py:269-281,380-391,747-749,1184,1312-1321``; branch decisions
``policies/pi07/low_level/modeling_pi07_low_level.py:93-191``).  They carry bytes, not tensors of the
model, so a library collective is the right tool here.
"""

from __future__ import annotations

from typing import Any, Callable

import torch
import torch.distributed as dist


def is_dist() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def rank() -> int:
    return dist.get_rank() if is_dist() else 0


def world_size() -> int:
    return dist.get_world_size() if is_dist() else 1


def is_main_process() -> bool:
    return rank() == 0


def is_local_main_process() -> bool:
    """Rank 0 of THIS node (``LOCAL_RANK``): the one that writes to node-local disks."""
    import os
    return int(os.environ.get("LOCAL_RANK", "0") or 0) == 0 if is_dist() else True


def wait_for_everyone() -> None:
    if is_dist():
        dist.barrier()


def gather_scalars(values: dict[str, torch.Tensor | float], device=None) -> dict[str, torch.Tensor]:
    """One all-gather for a whole dict of scalars: returns ``name -> (world,)`` tensors (row aligned)."""
    names = list(values)
    dev = device or next((v.device for v in values.values() if isinstance(v, torch.Tensor)), torch.device("cpu"))
    vec = torch.stack([torch.as_tensor(values[n], dtype=torch.float32, device=dev).reshape(()) for n in names])
    if not is_dist():
        return {n: vec[i:i + 1] for i, n in enumerate(names)}
    out = [torch.empty_like(vec) for _ in range(world_size())]
    dist.all_gather(out, vec)
    stacked = torch.stack(out)
    return {n: stacked[:, i] for i, n in enumerate(names)}


def gather_tensors(t: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """Concatenates per-rank ``(B, ...)`` tensors along dim 0 for every key (same B on all ranks)."""
    if not is_dist():
        return dict(t)
    out = {}
    for k, v in t.items():
        parts = [torch.empty_like(v) for _ in range(world_size())]
        dist.all_gather(parts, v.contiguous())
        out[k] = torch.cat(parts, 0)
    return out


def gather_ragged(t: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """Like :func:`gather_tensors` when the ranks hold DIFFERENT numbers of rows (the last shard of a sequential pass):
    the lengths are exchanged first, every rank pads to the longest, and the padding is cut out after the gather, so
    all keys stay row-aligned.  Every key of one rank must have the same number of rows."""
    if not is_dist():
        return dict(t)
    keys = sorted(t)
    n = int(t[keys[0]].shape[0]) if keys else 0
    dev = t[keys[0]].device if keys else torch.device("cpu")
    mine = torch.tensor([n], dtype=torch.long, device=dev)
    lens = [torch.zeros_like(mine) for _ in range(world_size())]
    dist.all_gather(lens, mine)
    lens = [int(x) for x in lens]
    longest = max(lens)
    out = {}
    for k in keys:
        v = t[k].contiguous()
        if v.shape[0] < longest:
            v = torch.cat([v, v.new_zeros((longest - v.shape[0], *v.shape[1:]))])
        parts = [torch.empty_like(v) for _ in range(world_size())]
        dist.all_gather(parts, v)
        out[k] = torch.cat([p_[:m] for p_, m in zip(parts, lens)], 0)
    return out


def reduce_sum(t: torch.Tensor) -> torch.Tensor:
    if is_dist():
        t = t.clone()
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t


def broadcast_object(obj: Any, src: int = 0) -> Any:
    if not is_dist():
        return obj
    box = [obj if rank() == src else None]
    dist.broadcast_object_list(box, src=src)
    return box[0]


def gather_object(obj: Any) -> list[Any]:
    if not is_dist():
        return [obj]
    out: list[Any] = [None] * world_size()
    dist.all_gather_object(out, obj)
    return out


def any_rank(flags: list[bool], device=None) -> list[bool]:
    """Element-wise OR across ranks of a list of booleans (one int32 all-reduce)."""
    if not is_dist():
        return list(flags)
    dev = device or (torch.device("cuda", torch.cuda.current_device())
                     if dist.get_backend() == "nccl" else torch.device("cpu"))
    t = torch.tensor([int(bool(f)) for f in flags], dtype=torch.int32, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return [bool(x) for x in t.tolist()]


def all_ranks_agree(value: Any) -> bool:
    vals = gather_object(value)
    return all(v == vals[0] for v in vals)


def on_main_process(fn: Callable, *args, sync: bool = True, **kwargs) -> Any:
    """Runs ``fn`` on rank 0 only and (``sync``) broadcasts its result; every path ends in a barrier."""
    result = fn(*args, **kwargs) if is_main_process() else None
    if sync:
        result = broadcast_object(result, 0)
    wait_for_everyone()
    return result
