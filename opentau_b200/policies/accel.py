"""``accel``: a flow-matching uncertainty proxy computed from the first Euler steps of a sample call.

``accel = sum_k ||v_k - v_{k-1}|| / sum_k ||v_k||`` over the first ``prefix`` velocity fields: a straight
flow (confident sample) keeps the velocity constant and scores near 0; a flow that bends scores high.
Only executed chunk rows (not frozen by real-time chunking, inside ``n_action_steps``) and real action
dims count.  Everything accumulates in fp32 on the device with no host synchronisation.  The feature is
off unless an entry point arms it with :func:`configure_accel` (reference
``src/opentau/policies/accel.py:111-863``).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
from torch import Tensor

MIN_PREFIX = 2


def default_prefix(num_steps: int) -> int:
    """Half of the Euler steps, at least :data:`MIN_PREFIX`."""
    return max(MIN_PREFIX, num_steps // 2)


def resolve_prefix(prefix: int | str | None, num_steps: int) -> int | None:
    """``None`` -> off; ``"auto"`` / ``0`` -> :func:`default_prefix`; else clamp into ``[2, num_steps]``."""
    if prefix is None:
        return None
    if isinstance(prefix, str):
        if prefix.lower() in ("auto", "default"):
            return min(num_steps, default_prefix(num_steps))
        prefix = int(prefix)
    if prefix == 0:
        return min(num_steps, default_prefix(num_steps))
    if prefix < MIN_PREFIX:
        raise ValueError(f"accel prefix must be >= {MIN_PREFIX}, got {prefix}")
    return min(int(prefix), num_steps)


def executed_row_mask(prefix_mask: Tensor, delay: Tensor | int, chunk_size: int, n_action_steps: int,
                      device) -> Tensor:
    """Rows that reach the robot: not frozen and inside ``[delay, delay + n_action_steps)``."""
    idx = torch.arange(chunk_size, device=device)[None, :]
    d = torch.as_tensor(delay, device=device).reshape(-1, 1) if not isinstance(delay, int) else delay
    return (~prefix_mask.to(device)) & (idx < d + n_action_steps)


def resolve_action_dim_mask(real_action_dim: Tensor | int | None, max_action_dim: int, batch: int,
                            device) -> Tensor | None:
    """``(B, action_dim)`` bool marking the dims that are real (not zero padding)."""
    if real_action_dim is None:
        return None
    r = torch.as_tensor(real_action_dim, device=device).reshape(-1, 1).expand(batch, 1)
    return torch.arange(max_action_dim, device=device)[None, :] < r


@dataclass(frozen=True)
class AccelProvenance:
    """What an ``accel`` value was measured with; thresholds fitted under one provenance are only
    comparable with observations under the same one."""

    policy_type: str
    num_steps: int
    prefix: int
    chunk_size: int
    n_action_steps: int
    action_dims: int

    def comparable_with(self, other: "AccelProvenance") -> bool:
        return self == other


def assert_comparable(fitted: AccelProvenance, observed: AccelProvenance) -> None:
    if not fitted.comparable_with(observed):
        raise ValueError(f"accel values are not comparable: fitted under {fitted}, observed under {observed}")


@dataclass
class AccelMeter:
    prefix: int
    batch_size: int
    device: torch.device
    dim_mask: Tensor | None = None
    record_trace: bool = False
    _num: Tensor = field(init=False, repr=False)
    _den: Tensor = field(init=False, repr=False)
    _prev: Tensor | None = field(default=None, init=False, repr=False)
    _mask: Tensor | None = field(default=None, init=False, repr=False)
    _steps: int = field(default=0, init=False)
    trace: list = field(default_factory=list, init=False, repr=False)

    def __post_init__(self):
        if self.prefix < MIN_PREFIX:
            raise ValueError(f"accel prefix must be >= {MIN_PREFIX}, got {self.prefix}.")
        self._num = torch.zeros(self.batch_size, dtype=torch.float32, device=self.device)
        self._den = torch.zeros(self.batch_size, dtype=torch.float32, device=self.device)
        if self.dim_mask is not None:
            self._mask = self.dim_mask.to(torch.float32)[:, None, :]

    def set_row_mask(self, row_mask: Tensor) -> None:
        rows = row_mask.to(torch.float32)[:, :, None]
        self._mask = rows if self._mask is None else rows * self._mask

    def update(self, v_t: Tensor) -> None:
        if self._steps >= self.prefix:
            return
        v = v_t.to(torch.float32)
        if self._mask is not None:
            v = v * self._mask
        v = v.flatten(1)
        n = torch.linalg.vector_norm(v, dim=1)
        self._den = self._den + n
        if self._prev is not None:
            self._num = self._num + torch.linalg.vector_norm(v - self._prev, dim=1)
        if self.record_trace:
            self.trace.append(n)
        self._prev = v
        self._steps += 1

    def value(self) -> Tensor:
        """``(B,)`` fp32; 0 where no velocity mass was seen."""
        return torch.where(self._den > 0, self._num / self._den.clamp_min(1e-12), torch.zeros_like(self._num))


def make_meter(policy, batch_size: int, device, real_action_dim=None) -> AccelMeter | None:
    prefix = getattr(policy, "_accel_prefix", None)
    if prefix is None:
        return None
    mask = resolve_action_dim_mask(real_action_dim, policy.config.max_action_dim, batch_size, device)
    return AccelMeter(prefix, batch_size, torch.device(device), mask)


def build_provenance(policy, prefix: int) -> AccelProvenance:
    c = policy.config
    feat = c.action_feature
    return AccelProvenance(c.type, c.num_steps, prefix, c.chunk_size, c.n_action_steps,
                           feat.shape[0] if feat is not None else c.max_action_dim)


def configure_accel(policy, prefix: int | str | None) -> AccelProvenance | None:
    """The only writer of the policy's accel setting: ``None`` disarms it."""
    resolved = resolve_prefix(prefix, policy.config.num_steps)
    policy._accel_prefix = resolved
    policy.last_accel = None
    policy.last_accel_provenance = build_provenance(policy, resolved) if resolved is not None else None
    return policy.last_accel_provenance
