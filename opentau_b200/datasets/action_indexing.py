"""Column selection and delta-action conversion for state / action vectors
(reference ``src/opentau/datasets/action_indexing.py:51-258``).

Two index spaces are in play and every function here says which one it takes:

* PARQUET space: columns of the raw ``state`` / ``action`` vectors stored with the dataset.  ``DatasetConfig``'s
  ``state_index``, ``action_index`` and ``delta_action_state_map`` are written in it.
* POST-INDEX space: positions in the vectors the dataset emits, after ``state_index`` / ``action_index`` have chosen
  and reordered columns.  The policy only ever sees these, so the map it stores to turn its outputs back into
  absolute actions lives here.

:func:`resolve_delta_map` is the one translation between the two; the dataset (which forms the deltas) and the mixture
metadata (which publishes the policy's map) both call it.

The delta itself follows the chunk-start convention: ONE state, the one observed when the chunk begins, is subtracted
from every step of the chunk on the mapped dims (``a'[k, i] = a[k, i] - state[j]``), so step ``k`` holds the cumulative
displacement and not a per-step increment.  Unmapped dims (an absolute gripper) pass through.
"""

from __future__ import annotations

import logging

import torch
from torch import Tensor

__all__ = ["add_chunk_start_state", "apply_column_index", "apply_delta_actions", "normalize_delta_map",
           "resolve_delta_map", "subtract_chunk_start_state", "undo_delta_actions"]


def apply_column_index(value: Tensor, index: list[int] | None, *, what: str = "vector", who: str = "dataset") -> Tensor:
    """``value[..., index]`` (PARQUET space, emission order); ``None`` returns ``value`` itself.  Every out-of-range
    column is named at once: the alternative is a shape error deep inside the policy."""
    if index is None:
        return value
    width = value.shape[-1]
    bad = [i for i in index if not 0 <= i < width]
    if bad:
        raise IndexError(f"{who}: {what}_index names column(s) {bad}, but the raw '{what}' has {width} column(s) "
                         f"(0..{width - 1})")
    return value.index_select(-1, torch.as_tensor(index, dtype=torch.long, device=value.device))


def normalize_delta_map(delta_map: dict | None) -> dict[int, int]:
    """Integer keys and values (JSON and CLI parsing produce strings)."""
    return {int(k): int(v) for k, v in (delta_map or {}).items()}


def resolve_delta_map(parquet_map: dict | None, action_index: list[int] | None, state_index: list[int] | None, *,
                      who: str = "dataset", action_dim: int | None = None, warn_unmapped: bool = True) -> dict[int, int]:
    """``{action column: state column}`` in PARQUET space -> ``{action position: state position}`` in POST-INDEX space.

    A mapped column that the matching index drops is an error (the config says "relative", the data would train
    absolute).  With ``action_dim`` (emitted width) known, kept dims that have no entry are listed in one warning."""
    pmap = normalize_delta_map(parquet_map)
    a_pos = None if action_index is None else {c: p for p, c in enumerate(action_index)}
    s_pos = None if state_index is None else {c: p for p, c in enumerate(state_index)}
    out: dict[int, int] = {}
    lost_actions, lost_states = [], []
    for a_col, s_col in sorted(pmap.items()):
        if a_pos is not None and a_col not in a_pos:
            lost_actions.append(a_col)
        elif s_pos is not None and s_col not in s_pos:
            lost_states.append((a_col, s_col))
        else:
            out[a_col if a_pos is None else a_pos[a_col]] = s_col if s_pos is None else s_pos[s_col]
    if lost_actions:
        raise ValueError(f"{who}: delta_action_state_map maps action column(s) {lost_actions} that "
                         f"action_index={action_index} does not keep; keep them or take them out of the map")
    if lost_states:
        raise ValueError(f"{who}: delta_action_state_map takes action column(s) {[a for a, _ in lost_states]} relative to "
                         f"state column(s) {[s for _, s in lost_states]}, which state_index={state_index} drops")
    if warn_unmapped and action_dim is not None:
        absolute = [p for p in range(action_dim) if p not in out]
        if absolute:
            logging.warning("%s: delta joint actions are on, but emitted action dim(s) %s have no entry in "
                            "delta_action_state_map and train as ABSOLUTE (%d of %d dims are relative); add them to the "
                            "map if that is not intended", who, absolute, len(out), action_dim)
    return out


def _offset(actions: Tensor, state: Tensor, delta_map: dict | None, sign: float) -> Tensor:
    """``actions (chunk, A)`` or ``(B, chunk, A)``; ``state (S,)`` / ``(B, S)``, or with a history axis
    ``(T, S)`` / ``(B, T, S)`` (same rank as ``actions``: the LAST step is the chunk's anchor).  New tensor."""
    dm = normalize_delta_map(delta_map)
    if not dm:
        return actions
    current = state[..., -1, :] if state.dim() == actions.dim() else state
    a_idx = sorted(dm)
    if a_idx[-1] >= actions.shape[-1] or max(dm.values()) >= current.shape[-1]:
        raise IndexError(f"delta map {dm} reaches outside the action / state widths "
                         f"{actions.shape[-1]} / {current.shape[-1]}")
    a_pos = torch.as_tensor(a_idx, dtype=torch.long, device=actions.device)
    s_pos = torch.as_tensor([dm[a] for a in a_idx], dtype=torch.long, device=actions.device)
    out = actions.clone()
    out[..., a_pos] += sign * current.to(device=out.device)[..., s_pos].unsqueeze(-2).to(out.dtype)
    return out


def subtract_chunk_start_state(actions: Tensor, state: Tensor, delta_map: dict | None) -> Tensor:
    """Absolute actions -> displacements from the chunk-start state on the mapped dims (POST-INDEX map)."""
    return _offset(actions, state, delta_map, -1.0)


def add_chunk_start_state(actions: Tensor, state: Tensor, delta_map: dict | None) -> Tensor:
    """Inverse of :func:`subtract_chunk_start_state`: what the policy emits -> absolute actions."""
    return _offset(actions, state, delta_map, 1.0)


apply_delta_actions = subtract_chunk_start_state
undo_delta_actions = add_chunk_start_state
