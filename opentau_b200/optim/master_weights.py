"""``MasterWeightOptimizer``: fp32 master copies for bf16 parameters around any torch optimizer
(reference ``src/opentau/optim/master_weights.py:38-439``).

The training engine keeps sharded fp32 masters inside its fused step; this wrapper serves code that drives a plain
``torch.optim`` optimizer itself (scripts, notebooks, the generic optimizer factory): gradients are copied to fp32,
the wrapped optimizer steps the masters, the bf16 parameters are refreshed by rounding.
"""

from __future__ import annotations

from typing import Any, Callable

import torch
from torch import Tensor


class MasterWeightOptimizer:
    def __init__(self, params, optimizer_factory: Callable[[list[Tensor]], torch.optim.Optimizer]):
        self.model_params = [p for p in params if p.requires_grad]
        self.masters = [p.detach().clone().float().requires_grad_(True) for p in self.model_params]
        self.optimizer = optimizer_factory(self.masters)

    @classmethod
    def from_existing(cls, optimizer: torch.optim.Optimizer) -> "MasterWeightOptimizer":
        """Re-targets an optimizer built on the bf16 parameters at fresh fp32 masters (same hyper-parameters)."""
        groups = optimizer.param_groups
        params = [p for g in groups for p in g["params"]]
        hyper = {k: v for k, v in groups[0].items() if k != "params"}
        return cls(params, lambda masters: type(optimizer)(masters, **hyper))

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.model_params:
            p.grad = None if set_to_none else (p.grad.zero_() if p.grad is not None else None)
        self.optimizer.zero_grad(set_to_none=set_to_none)

    def _sync_grads(self) -> None:
        for p, m in zip(self.model_params, self.masters):
            m.grad = None if p.grad is None else p.grad.detach().float()

    def clip_grad_norm_(self, max_norm: float) -> Tensor:
        self._sync_grads()
        with_grad = [m for m in self.masters if m.grad is not None]
        norm = torch.nn.utils.clip_grad_norm_(with_grad, max_norm) if with_grad else torch.zeros(())
        self._clipped = True
        return norm

    @torch.no_grad()
    def step(self) -> None:
        if not getattr(self, "_clipped", False):
            self._sync_grads()
        self._clipped = False
        self.optimizer.step()
        for p, m in zip(self.model_params, self.masters):
            p.copy_(m.to(p.dtype))

    @torch.no_grad()
    def rebuild_masters_from_live(self) -> None:
        """After loading bf16 weights (or moving devices) the masters restart from the live parameters."""
        for p, m in zip(self.model_params, self.masters):
            if m.device != p.device:
                m.data = p.detach().float().clone()
            else:
                m.copy_(p.float())

    def state_dict(self) -> dict[str, Any]:
        return {"optimizer": self.optimizer.state_dict(), "masters": [m.detach().cpu() for m in self.masters]}

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        self.optimizer.load_state_dict(sd["optimizer"])
        for m, s in zip(self.masters, sd["masters"]):
            m.data.copy_(s.to(m.device))
