"""``PerGroupLinear``: a linear layer with one independent ``(weight, bias)`` per group (per robot embodiment /
dataset head), selected per sample (reference ``src/opentau/policies/layers.py:37-127``).

Parameters are an ``nn.Linear``'s with a leading group axis — ``weight (G, out, in)``, ``bias (G, out)`` — so
state-dict keys equal those of a plain linear layer and a legacy checkpoint promotes by prepending the axis
(:func:`promote_linear_state`).  ``G == 1`` is a plain GEMM.  For ``G > 1`` samples are bucketed by group and each
bucket is one GEMM on the hand-written kernel path, instead of materialising a ``(B, out, in)`` gathered weight.
"""

from __future__ import annotations

import math

import torch
from torch import Tensor, nn

from .. import ops


class PerGroupLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, num_groups: int, bias: bool = True):
        super().__init__()
        if num_groups < 1:
            raise ValueError(f"num_groups must be >= 1, got {num_groups}.")
        self.in_features, self.out_features, self.num_groups = in_features, out_features, num_groups
        self.weight = nn.Parameter(torch.empty(num_groups, out_features, in_features))
        if bias:
            self.bias = nn.Parameter(torch.empty(num_groups, out_features))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        for g in range(self.num_groups):
            nn.init.kaiming_uniform_(self.weight[g], a=math.sqrt(5))
            if self.bias is not None:
                bound = 1.0 / math.sqrt(self.in_features) if self.in_features > 0 else 0.0
                nn.init.uniform_(self.bias[g], -bound, bound)

    def forward(self, x: Tensor, group_index: Tensor | None = None) -> Tensor:
        if self.num_groups == 1:
            return ops.linear(x.to(self.weight.dtype), self.weight[0], None if self.bias is None else self.bias[0])
        if group_index is None:
            group_index = torch.zeros(x.shape[0], dtype=torch.long, device=x.device)
        out = x.new_empty(*x.shape[:-1], self.out_features, dtype=self.weight.dtype)
        xw = x.to(self.weight.dtype)
        for g in torch.unique(group_index).tolist():
            sel = (group_index == g).nonzero(as_tuple=True)[0]
            out[sel] = ops.linear(xw[sel], self.weight[g], None if self.bias is None else self.bias[g])
        return out

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"num_groups={self.num_groups}, bias={self.bias is not None}")


def promote_linear_state(state: dict[str, Tensor], prefix: str, num_groups: int) -> dict[str, Tensor]:
    """Turns ``<prefix>.weight (out, in)`` / ``.bias (out)`` of a plain linear layer into per-group tensors by
    repeating them over ``num_groups`` (every group starts from the shared map)."""
    out = dict(state)
    for suffix, rank in (("weight", 2), ("bias", 1)):
        k = f"{prefix}.{suffix}"
        if k in out and out[k].dim() == rank:
            out[k] = out[k].unsqueeze(0).repeat(num_groups, *([1] * rank)).contiguous()
    return out
