"""Column selection and delta-action conversion for state / action vectors
(reference ``src/opentau/datasets/action_indexing.py:27-220``).

``state_index`` / ``action_index`` subset and reorder the raw columns.  ``delta_action_state_map`` maps an action
dim (after indexing) to the state dim (after indexing) it is relative to: ``a'[t, i] = a[t, i] - state[j]`` for
every step of the chunk, with the state of the CURRENT frame.
"""

from __future__ import annotations

import torch
from torch import Tensor


def apply_column_index(x: Tensor, index: list[int] | None) -> Tensor:
    if index is None:
        return x
    if max(index) >= x.shape[-1]:
        raise IndexError(f"column index {max(index)} out of range for a vector of width {x.shape[-1]}")
    return x[..., torch.as_tensor(index, dtype=torch.long)]


def normalize_delta_map(delta_map: dict | None) -> dict[int, int]:
    return {int(k): int(v) for k, v in (delta_map or {}).items()}


def apply_delta_actions(actions: Tensor, state: Tensor, delta_map: dict | None) -> Tensor:
    """``actions (T, A)``, ``state (S,)`` or ``(Th, S)`` (last row = current frame)."""
    dm = normalize_delta_map(delta_map)
    if not dm:
        return actions
    cur = state[-1] if state.dim() == 2 else state
    out = actions.clone()
    for a_dim, s_dim in dm.items():
        if a_dim >= out.shape[-1] or s_dim >= cur.shape[-1]:
            raise IndexError(f"delta map entry {a_dim}->{s_dim} outside action/state widths "
                             f"{out.shape[-1]}/{cur.shape[-1]}")
        out[..., a_dim] = out[..., a_dim] - cur[s_dim]
    return out


def undo_delta_actions(actions: Tensor, state: Tensor, delta_map: dict | None) -> Tensor:
    """Inverse of :func:`apply_delta_actions` for ``actions (..., T, A)`` and the current ``state (..., S)``."""
    dm = normalize_delta_map(delta_map)
    if not dm:
        return actions
    out = actions.clone()
    for a_dim, s_dim in dm.items():
        out[..., a_dim] = out[..., a_dim] + state[..., s_dim].unsqueeze(-1)
    return out
