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


@dataclass
class FlatGroup:
    dtype: torch.dtype
    params: list[nn.Parameter]
    names: list[str]
    offsets: list[int]
    numel: int                 # padded total
    data: Tensor               # flat parameter buffer
    grad: Tensor               # flat gradient buffer (same dtype)


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class FlatParamStore:
    """Re-homes the trainable parameters of ``module`` into flat buffers on ``device``."""

    def __init__(self, module: nn.Module, device: torch.device | str, pad_to: int = 1,
                 allocator=None):
        self.device = torch.device(device)
        by_dtype: dict[torch.dtype, list[tuple[str, nn.Parameter]]] = {}
        seen: set[int] = set()
        for name, p in module.named_parameters():
            if not p.requires_grad or id(p) in seen:
                continue
            seen.add(id(p))
            by_dtype.setdefault(p.dtype, []).append((name, p))
        self.groups: list[FlatGroup] = []
        alloc = allocator or (lambda n, dt: torch.zeros(n, dtype=dt, device=self.device))
        for dtype, items in by_dtype.items():
            offsets, off = [], 0
            for _, p in items:
                offsets.append(off)
                off = _round_up(off + p.numel(), ALIGN_ELEMS)
            total = _round_up(off, ALIGN_ELEMS * max(1, pad_to))
            data = alloc(total, dtype)
            grad = alloc(total, dtype)
            for (name, p), o in zip(items, offsets):
                view = data[o:o + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.main_grad = grad[o:o + p.numel()].view(p.shape)
                p.grad = None
            self.groups.append(FlatGroup(dtype, [p for _, p in items], [n for n, _ in items], offsets, total,
                                         data, grad))
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
            g.grad.zero_()
            for p in g.params:
                p.grad = None

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
                 "params": [{"name": n, "shape": list(p.shape), "offset": o}
                            for n, p, o in zip(g.names, g.params, g.offsets)]} for g in self.groups]

    @property
    def num_trainable(self) -> int:
        return sum(p.numel() for g in self.groups for p in g.params)
