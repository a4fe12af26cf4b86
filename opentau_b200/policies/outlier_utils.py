"""Detection of badly normalised state / action dimensions (reference ``src/opentau/policies/outlier_utils.py:30-201``).

A normalised value far from unit scale nearly always means broken statistics (a near-constant dim with a tiny std)
or corrupt data.  ``detect_state_action_outliers`` is pure and collective-free — it inspects one local batch and
returns plain-Python records, so every rank issues the same collectives whatever its data holds; the training loop
merges the records across ranks and logs each offender once (``log_outlier_records``).
"""

from __future__ import annotations

import logging
from typing import Any

import torch
from torch import Tensor


def _per_sample(value: Any, i: int) -> Any:
    if isinstance(value, list):
        return value[i]
    if torch.is_tensor(value):
        return int(value[i])
    return value


def _attended_steps_mask(key: str, t: Tensor, batch: dict[str, Any]) -> Tensor | None:
    """``(B, T)`` bool of the steps the model actually attends to (padded history / padded action steps excluded; the
    current state frame always kept), or None to scan everything."""
    if t.dim() < 3:
        return None
    if key == "state":
        pad = batch.get("obs_history_is_pad")
        if pad is not None and (pad.dim() != 2 or pad.shape[1] != t.shape[1]):
            return None
        keep = torch.zeros(t.shape[:2], dtype=torch.bool, device=t.device) if pad is None else ~pad.bool()
        keep = keep.clone()
        keep[:, -1] = True
        return keep
    if key == "actions":
        pad = batch.get("action_is_pad")
        if pad is None or pad.dim() != 2 or pad.shape[1] != t.shape[1]:
            return None
        return ~pad.bool()
    return None


def detect_state_action_outliers(batch: dict[str, Any], threshold: float | None) -> list[dict[str, Any]]:
    """One record ``{key, source, dim, value, episode, frame}`` per offending ``(source, key, dim)``: the largest
    ``|normalised value|`` above ``threshold`` and where it came from.  ``threshold`` None or <= 0 disables."""
    if threshold is None or threshold <= 0:
        return []
    per_key: dict[str, Tensor] = {}
    for key in ("state", "actions"):
        t = batch.get(key)
        if t is None:
            continue
        t = t.detach().abs().float()
        keep = _attended_steps_mask(key, t, batch)
        if keep is not None:
            t = t * keep[:, :, None].to(t.dtype)
        per_key[key] = t.reshape(t.shape[0], -1, t.shape[-1]).amax(dim=1)
    if not per_key or not bool(torch.cat([(v > threshold).flatten() for v in per_key.values()]).any()):
        return []
    src = batch.get("dataset_repo_id", batch.get("source"))
    ep, fr = batch.get("episode_index"), batch.get("frame_index")
    records: list[dict[str, Any]] = []
    for key, pdm in per_key.items():
        pdm = pdm.cpu()
        worst: dict[tuple, tuple[float, int]] = {}
        for s_i, d in torch.nonzero(pdm > threshold, as_tuple=False).tolist():
            tup = (_per_sample(src, s_i), key, d)
            val = float(pdm[s_i, d])
            if tup not in worst or val > worst[tup][0]:
                worst[tup] = (val, s_i)
        for (source, k, d), (val, s_i) in worst.items():
            records.append({"key": k, "source": source, "dim": d, "value": val, "episode": _per_sample(ep, s_i),
                            "frame": _per_sample(fr, s_i)})
    return records


_ALREADY_WARNED: set[tuple] = set()


def log_outlier_records(records: list[dict[str, Any]], threshold: float, seen: set | None = None) -> int:
    """Logs each ``(source, key, dim)`` once per process lifetime; returns how many were new."""
    seen = _ALREADY_WARNED if seen is None else seen
    new = 0
    for r in sorted(records, key=lambda r: -r["value"]):
        tup = (r["source"], r["key"], r["dim"])
        if tup in seen:
            continue
        seen.add(tup)
        new += 1
        logging.warning("normalised %s dim %d of %s reaches |%.1f| (> %.1f) at episode %s frame %s: check the "
                        "normalisation statistics of this dimension", r["key"], r["dim"], r["source"], r["value"],
                        threshold, r["episode"], r["frame"])
    return new


def log_outlier_records_distributed(records: list[dict[str, Any]], threshold: float) -> int:
    """Every rank contributes its records (an all-reduce of the count decides, identically on all ranks, whether the
    object gather runs); rank 0 logs."""
    from ..parallel import control
    n = torch.tensor(float(len(records)))
    total = float(control.reduce_sum(n))
    if total == 0:
        return 0
    merged = [r for part in control.gather_object(records) for r in part]
    return log_outlier_records(merged, threshold) if control.is_main_process() else 0
