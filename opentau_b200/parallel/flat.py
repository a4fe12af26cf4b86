"""Flat parameter / gradient storage.

All trainable parameters of a dtype live back to back in one buffer, and so do their gradients
(``param.main_grad`` views).  That is what makes the data-parallel step three launches instead of
thousands: one reduce-scatter over the gradient buffer, one fused AdamW over this rank's shard of
fp32 masters, one all-gather of the refreshed bf16 parameters — or a single fused peer-memory
kernel doing all three (``parallel/comm.py``).

The reference reaches the same state through ``accelerate`` wrappers: DDP buckets + a per-tensor
fp32 master optimizer (OpenTau ``src/opentau/optim/master_weights.py:38-297``) or DeepSpeed ZeRO /
FSDP flat parameters (``configs/examples/accelerate_*.yaml``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import Tensor, nn

ALIGN_ELEMS = 128  # every parameter starts on a 256-byte boundary (TMA needs 16 B; shards split cleanly)
DEFAULT_BUCKET_ELEMS = 48 * 1024 * 1024   # ~ one Gemma-2B decoder layer's attention + half its MLP in bf16


@dataclass
class Bucket:
    """A contiguous run ``[lo, hi)`` of whole parameters of one flat group.  It is the unit of gradient
    communication: once every parameter inside has its gradient, the bucket is reduced while the backward pass of
    earlier layers is still running.  ``hi - lo`` is a multiple of ``ALIGN_ELEMS * world``, so every rank owns an
    equal, 256-byte aligned slice of every bucket."""
    index: int                 # global index over all groups (flag slot, partial-sum slot)
    group: int
    lo: int
    hi: int
    first_param: int           # parameters [first_param, last_param) of the group live in this bucket
    last_param: int

    @property
    def numel(self) -> int:
        return self.hi - self.lo


@dataclass
class FlatGroup:
    dtype: torch.dtype
    params: list[nn.Parameter]
    names: list[str]
    offsets: list[int]
    numel: int                 # padded total
    data: Tensor               # flat parameter buffer
    grad: Tensor               # flat gradient buffer (same dtype)
    buckets: list[Bucket] | None = None


def _late_gradient(name: str) -> bool:
    """Parameters whose gradient arrives only at the very end of a tower's backward pass (the adaptive-norm
    projections of ALL layers are one stacked product computed before the first layer).  They are laid out behind
    the other parameters so they do not hold back the buckets of the layers they belong to."""
    return "layernorm.dense." in name or name.endswith("norm.dense.weight") or name.endswith("norm.dense.bias")


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class FlatParamStore:
    """Re-homes the trainable parameters of ``module`` into flat buffers on ``device``."""

    def __init__(self, module: nn.Module, device: torch.device | str, pad_to: int = 1,
                 allocator=None, bucket_elems: int = DEFAULT_BUCKET_ELEMS, bucket_key=None):
        """``bucket_key(name) -> str`` (optional) names the bucket of every parameter: parameters with one key are
        laid out together as ONE bucket whatever its size (keys in order of first appearance).  The
        parameter-sharded engine uses it to make a bucket the unit it gathers before a layer runs."""
        self.device = torch.device(device)
        self.world = max(1, pad_to)
        self.bucket_keys: list[str] = []
        by_dtype: dict[torch.dtype, list[tuple[str, nn.Parameter]]] = {}
        seen: set[int] = set()
        for name, p in module.named_parameters():
            if not p.requires_grad or id(p) in seen:
                continue
            seen.add(id(p))
            by_dtype.setdefault(p.dtype, []).append((name, p))
        self.groups: list[FlatGroup] = []
        alloc = allocator or (lambda n, dt: torch.zeros(n, dtype=dt, device=self.device))
        self.buckets: list[Bucket] = []
        step = ALIGN_ELEMS * self.world
        for gi, (dtype, items) in enumerate(by_dtype.items()):
            keys = None
            if bucket_key is not None:
                order: dict[str, int] = {}
                for name, _ in items:
                    order.setdefault(bucket_key(name), len(order))
                items.sort(key=lambda it: order[bucket_key(it[0])])  # stable: one run of parameters per key
                keys = [bucket_key(name) for name, _ in items]
            else:
                items.sort(key=lambda it: _late_gradient(it[0]))     # stable: late-gradient parameters go last
            offsets, off = [], 0
            buckets: list[Bucket] = []
            b_lo, b_first = 0, 0
            for pi, (_, p) in enumerate(items):
                close = (keys[pi] != keys[pi - 1]) if (keys is not None and pi > 0) else \
                    (keys is None and off - b_lo >= bucket_elems)
                if close:                                            # close the bucket in front of this parameter
                    if keys is not None:
                        self.bucket_keys.append(keys[pi - 1])
                    off = _round_up(off, step)
                    buckets.append(Bucket(len(self.buckets) + len(buckets), gi, b_lo, off, b_first, pi))
                    b_lo, b_first = off, pi
                offsets.append(off)
                off = _round_up(off + p.numel(), ALIGN_ELEMS)
            total = _round_up(off, step)
            if keys is not None:
                self.bucket_keys.append(keys[-1])
            buckets.append(Bucket(len(self.buckets) + len(buckets), gi, b_lo, total, b_first, len(items)))
            self.buckets += buckets
            data = alloc(total, dtype)
            grad = alloc(total, dtype)
            for (name, p), o in zip(items, offsets):
                view = data[o:o + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.main_grad = grad[o:o + p.numel()].view(p.shape)
                p.grad = None
            self.groups.append(FlatGroup(dtype, [p for _, p in items], [n for n, _ in items], offsets, total,
                                         data, grad, buckets))
        # everything else (frozen parameters, buffers) simply moves to the device
        for p in module.parameters():
            if not p.requires_grad and p.device != self.device:
                p.data = p.data.to(self.device)
        for mod in module.modules():
            for k, b in list(mod._buffers.items()):
                if b is not None and b.device != self.device:
                    mod._buffers[k] = b.to(self.device)

    def zero_grad(self) -> None:
        for g in self.groups:
            if g.grad.is_cuda:
                from ..ops import cuda_ops
                cuda_ops.zero_(g.grad)
            else:
                g.grad.zero_()
            for p in g.params:
                p.grad = None

    def bucket_of_param(self) -> dict[int, Bucket]:
        """``id(parameter) -> bucket``."""
        out = {}
        for g in self.groups:
            for b in g.buckets:
                for p in g.params[b.first_param:b.last_param]:
                    out[id(p)] = b
        return out

    def fold_autograd_grads(self) -> None:
        """Adds gradients that autograd delivered in ``.grad`` (ops without a fused sink) into the
        flat buffer, so the flat gradient is the complete gradient."""
        for g in self.groups:
            for p in g.params:
                if p.grad is not None:
                    p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                    p.grad = None

    def layout(self) -> list[dict]:
        """Name / shape / offset of every parameter inside each flat group: what an offline tool needs to turn the
        per-rank optimizer shards back into named tensors."""
        return [{"dtype": str(g.dtype).replace("torch.", ""), "numel": g.numel,
                 "buckets": [[b.lo, b.hi] for b in g.buckets],
                 "params": [{"name": n, "shape": list(p.shape), "offset": o}
                            for n, p, o in zip(g.names, g.params, g.offsets)]} for g in self.groups]

    @property
    def num_trainable(self) -> int:
        return sum(p.numel() for g in self.groups for p in g.params)
