"""Turn evaluation rollouts into a LeRobot dataset (one episode per sub-environment, cut at its first ``done``).

The reference does this for LIBERO evaluations (``src/opentau/utils/libero_dataset_recorder.py:196-460``:
``consolidate_task_result`` writes parquet / metadata by hand for the fixed LIBERO schema, ``aggregate_task_results``
merges several results).  Here the input is what ``scripts.eval.rollout(..., return_observations=True)`` returns for any
environment, the output goes through the regular dataset recorder (so statistics, task table and video / image storage
are the ordinary ones), and the per-episode outcome is kept as ``success`` / ``sum_reward`` in ``meta/episodes.jsonl``
through the metadata attachment tool: the result can be fed straight back into training (success-filtered behaviour
cloning, value / advantage labelling).
"""

from __future__ import annotations

from pathlib import Path
from typing import Any

import numpy as np
import torch


def aggregate_rollouts(results: list[dict[str, Any]]) -> dict[str, Any]:
    """Concatenates rollout dicts along the batch axis; shorter rollouts are padded in time with ``done = True``."""
    T = max(r["done"].shape[1] for r in results)

    def pad(x: torch.Tensor, value) -> torch.Tensor:
        if x.shape[1] == T:
            return x
        fill = torch.full((x.shape[0], T - x.shape[1], *x.shape[2:]), value, dtype=x.dtype)
        return torch.cat([x, fill], 1)

    out = {"action": torch.cat([pad(r["action"], 0) for r in results]),
           "reward": torch.cat([pad(r["reward"], 0) for r in results]),
           "success": torch.cat([pad(r["success"], False) for r in results]),
           "done": torch.cat([pad(r["done"], True) for r in results]), "observation": []}
    for t in range(T):
        step: dict[str, Any] = {}
        for r in results:
            obs = r["observation"][min(t, len(r["observation"]) - 1)]
            for k, v in obs.items():
                step.setdefault(k, []).append(v)
        out["observation"].append({k: torch.cat(v) for k, v in step.items()})
    out["prompts"] = [p for r in results for p in r.get("prompts", [""] * r["done"].shape[0])]
    return out


def record_rollouts(data: dict[str, Any], output_dir: str | Path, fps: int, prompts: list[str] | None = None,
                    repo_id: str | None = None, robot_type: str = "sim", only_successful: bool = False,
                    use_videos: bool = False) -> dict[str, Any]:
    """``data``: one rollout (or ``aggregate_rollouts`` of several).  Returns ``{"episodes", "frames", "successes"}``."""
    from ..datasets.lerobot_dataset import LeRobotDataset
    from ..scripts.attach_metadata import attach
    obs0 = data["observation"][0]
    cams = sorted(k for k in obs0 if k.startswith("camera"))
    B, A = data["action"].shape[0], data["action"].shape[2]
    prompts = prompts or data.get("prompts") or [""] * B
    feats: dict[str, dict] = {"observation.state": {"dtype": "float32", "shape": (obs0["state"].shape[-1],), "names": None},
                              "action": {"dtype": "float32", "shape": (A,), "names": None}}
    for c in cams:
        _, C, H, W = obs0[c].shape
        feats[f"observation.images.{c}"] = {"dtype": "video" if use_videos else "image", "shape": (H, W, C),
                                            "names": ["height", "width", "channel"]}
    out = Path(output_dir)
    ds = LeRobotDataset.create(repo_id or out.name, fps=fps, root=out, robot_type=robot_type, features=feats,
                               use_videos=use_videos, image_writer_threads=2)
    done = data["done"].bool()
    T = done.shape[1]
    first_done = torch.where(done.any(1), done.int().argmax(1), torch.full((B,), T - 1))
    outcomes: dict[str, dict] = {}
    frames = 0
    for b in range(B):
        n = int(first_done[b]) + 1
        success = bool(data["success"][b, :n].any())
        if only_successful and not success:
            continue
        for t in range(n):
            o = data["observation"][t]
            frame = {"observation.state": o["state"][b].float().numpy(), "action": data["action"][b, t].float().numpy(),
                     "task": prompts[b]}
            for c in cams:
                img = (o[c][b].float().clamp(0, 1) * 255).round().byte().permute(1, 2, 0).numpy()
                frame[f"observation.images.{c}"] = np.ascontiguousarray(img)
            ds.add_frame(frame)
        ds.save_episode()
        outcomes[str(len(outcomes))] = {"success": success, "sum_reward": float(data["reward"][b, :n].sum())}
        frames += n
    ds.stop_image_writer()
    if outcomes:
        attach(out, {"episodes": outcomes})
    return {"episodes": len(outcomes), "frames": frames, "successes": sum(o["success"] for o in outcomes.values())}
