"""``opentau-eval``: closed-loop rollouts of a policy in (vectorised) environments.

Pipeline and result schema follow the reference (``src/opentau/scripts/eval.py:85-1567``): ``rollout`` steps a vector
environment until every sub-environment finished once, ``eval_policy`` repeats rollouts until ``n_episodes`` are
collected and reports per-episode ``sum_reward / max_reward / success / seed`` and the aggregate
``avg_sum_reward / avg_max_reward / pc_success / eval_s / eval_ep_s``, ``eval_policy_all`` walks the task groups
with tasks dealt round-robin to the ranks, and ``consolidate_eval_info`` merges the per-rank results into
``eval_info.json``.  Outputs built from frame ARRAYS need no graphics stack and are here too: per-episode clips and
the tiled ``grid_summary.mp4`` with a green / red border per tile for success / failure
(``eval.py:669-690, 793-952``), the goal-frame harvest of successful episodes keyed by scene seed
(``eval.py:475-484, 600-633``) and the per-chunk accel streams of a policy that publishes ``last_accel``
(``eval.py:466-471, 553-560``).  Frames come from the environments' ``render()`` (the headless ``fake`` environment
draws on the CPU); simulators that need a GL context are unavailable here.
"""

from __future__ import annotations

import json
import logging
import time
from pathlib import Path
from typing import Any

import numpy as np
import torch
from torch import Tensor

from ..configs import parser
from ..configs.deployment import tag_norm_head
from ..configs.train import TrainPipelineConfig
from ..envs.configs import EnvConfig
from ..envs.factory import make_envs
from ..envs.utils import (add_envs_task, add_eval_metadata, add_subgoal_images, check_env_attributes_and_types, close_envs,
                          preprocess_observation)
from ..parallel import control


def resolve_env_config(env: Any) -> EnvConfig:
    if isinstance(env, EnvConfig):
        return env
    if isinstance(env, dict):
        from ..configs.codec import decode
        d = dict(env)
        return decode(EnvConfig.get_choice_class(d.pop("type")), d, "env")      # nested blocks (metadata) included
    raise TypeError(f"cannot build an environment from {type(env).__name__}")


def _rank_seed_offset(rank: int, decorrelate: bool, per_rank_span: int = 100_003) -> int:
    """Added to every episode seed of a rank.  Off (the default): 0, every rank seeds alike, so the scene that a
    ``(task, episode)`` maps to does not depend on the number of GPUs or nodes.  On: rank ``r`` owns the block
    ``[r * span, (r + 1) * span)`` of the seed line, where ``span`` is exactly the number of seeds one rank consumes
    (batches x environments): the blocks tile the line, no gap, no overlap, however many episodes a rank runs.  ``rank``
    is the GLOBAL rank (a node-local one would alias across nodes).  Adjacent seeds are fine: each goes through a
    seed-sequence hash (reference ``src/opentau/scripts/eval.py:375-411``)."""
    return rank * per_rank_span if decorrelate else 0


def validate_eval_input_resolution(cfg) -> None:
    """Environment frames arrive at exactly ``cfg.resolution``.  With a resize target on the policy a mismatch only
    repeats the checkpoint's own double letterbox (a warning at construction); with NO resize target
    (``resize_imgs_with_padding`` null) nothing would correct the frames and the tower would silently run at another
    geometry than it was trained at: an error, unless ``policy.skip_input_resolution_check`` is set
    (reference ``src/opentau/scripts/eval.py:1049-1092``)."""
    pol = cfg.policy
    expected = getattr(pol, "input_image_size", None)
    if expected is None or tuple(cfg.resolution) == tuple(expected) \
            or getattr(pol, "resize_imgs_with_padding", None) is not None:
        return
    if pol.skip_input_resolution_check:
        logging.warning("resolution=%s differs from the policy's bound input resolution %s with "
                        "resize_imgs_with_padding=null; proceeding because skip_input_resolution_check=true",
                        tuple(cfg.resolution), tuple(expected))
        return
    raise ValueError(f"resolution={tuple(cfg.resolution)} but the policy was trained at {tuple(expected)} with "
                     "resize_imgs_with_padding=null (native pass-through): environment frames would reach the vision "
                     "tower at the wrong geometry with nothing to correct them.  Set resolution to match the checkpoint, "
                     "or policy.skip_input_resolution_check=true to proceed anyway.")


def collect_grid_summary_videos(videos_dir: Path) -> list[tuple[str, str]]:
    """Sorted ``(task name, path)`` of every ``grid_summary.mp4`` below ``videos_dir`` (for the experiment tracker); the
    task name is the folder name without a trailing ``_rank<N>``, so the keys stay the same when the number of GPUs
    changes (each task is evaluated on exactly one rank).  Per-episode clips are not listed."""
    import re
    videos_dir = Path(videos_dir)
    if not videos_dir.exists():
        return []
    return sorted((re.sub(r"_rank\d+$", "", g.parent.name), str(g)) for g in videos_dir.rglob("grid_summary.mp4"))


def rollout(env, policy, seeds: list[int] | None = None, cfg=None, device=None, return_observations: bool = False,
            extra_batch: dict[str, Any] | None = None, subgoal_generator=None, render_callback=None,
            capture_last_frames: bool = False) -> dict[str, Tensor]:
    """One batch of episodes.  Returns ``action (B,T,A)``, ``reward (B,T)``, ``success (B,T)``, ``done (B,T)``.
    ``subgoal_generator`` (``envs.subgoal``) pins one subgoal per sub-environment at the reset and feeds it to the
    policy at every step.  ``render_callback(env)`` is called after the reset and after every step (video frames).
    ``capture_last_frames``: ``last_frames[b]`` = the raw camera images ``{camera key: uint8 HWC}`` of episode
    ``b``'s final observation before the environment reset itself.  A policy that publishes ``last_accel`` after
    computing a chunk adds ``accel``: one list of values per episode, cut at the episode's end."""
    device = device or next(policy.parameters()).device
    policy.reset()
    obs, _ = env.reset(seed=seeds)
    check_env_attributes_and_types(env)
    if subgoal_generator is not None:
        subgoal_generator.start_episode(list(add_envs_task(env, preprocess_observation(obs, cfg))["prompt"]), seeds)
    max_steps = int(env.call("_max_episode_steps")[0])
    done = np.zeros(env.num_envs, dtype=bool)
    all_a, all_r, all_s, all_d, all_o = [], [], [], [], []
    last_frames: list[dict | None] = [None] * env.num_envs
    accel: list[list[float]] = [[] for _ in range(env.num_envs)]
    seen_accel = None
    step = 0
    if render_callback is not None:
        render_callback(env)
    while not done.all() and step < max_steps:
        if capture_last_frames:
            cams = _raw_cameras(obs)
            for b in range(env.num_envs):
                if not done[b]:
                    last_frames[b] = {k: v[b] for k, v in cams.items()}
        batch = preprocess_observation(obs, cfg)
        batch = add_envs_task(env, batch)
        if cfg is not None and getattr(cfg, "env", None) is not None:
            batch = add_eval_metadata(batch, resolve_env_config(cfg.env))
        batch = add_subgoal_images(batch, subgoal_generator)
        batch = {k: (v.to(device) if isinstance(v, Tensor) else v) for k, v in batch.items()}
        if extra_batch:
            batch.update(extra_batch)
        tag_norm_head(batch, getattr(cfg, "eval", None))
        if return_observations:
            all_o.append({k: v.cpu() for k, v in batch.items() if isinstance(v, Tensor)})
        with torch.inference_mode():
            action = policy.select_action(batch)
        cur = getattr(policy, "last_accel", None)
        if cur is not None and cur is not seen_accel:            # a new chunk was computed in this call
            seen_accel = cur
            vals = torch.as_tensor(cur).float().reshape(-1).tolist()
            for b in range(env.num_envs):
                if not done[b]:
                    accel[b].append(vals[b if len(vals) == env.num_envs else 0])
        a = action.float().cpu().numpy()
        obs, reward, terminated, truncated, info = env.step(a)
        if render_callback is not None:
            render_callback(env)
        if "final_info" in info:
            succ = np.array([bool(f["is_success"]) if f is not None else False for f in info["final_info"]])
        else:
            succ = np.asarray(info.get("is_success", np.zeros(env.num_envs, bool)))
        done = done | terminated | truncated
        all_a.append(torch.from_numpy(a)), all_r.append(torch.from_numpy(np.asarray(reward, np.float32)))
        all_s.append(torch.from_numpy(succ.astype(bool))), all_d.append(torch.from_numpy(done.copy()))
        step += 1
    out = {"action": torch.stack(all_a, 1), "reward": torch.stack(all_r, 1), "success": torch.stack(all_s, 1),
           "done": torch.stack(all_d, 1)}
    if return_observations:
        out["observation"] = all_o
    if capture_last_frames:
        out["last_frames"] = last_frames
    if seen_accel is not None:
        out["accel"] = accel
        prov = getattr(policy, "last_accel_provenance", None)
        out["accel_provenance"] = prov.to_dict() if hasattr(prov, "to_dict") else prov     # JSON-ready
    return out


def _raw_cameras(obs: dict) -> dict[str, np.ndarray]:
    """uint8 ``(B, H, W, C)`` camera arrays of a raw vector observation (``pixels`` may be one array or a dict)."""
    px = obs.get("pixels") if isinstance(obs, dict) else None
    if px is None:
        return {}
    if isinstance(px, dict):
        return {str(k): np.asarray(v) for k, v in px.items()}
    return {"camera0": np.asarray(px)}


def write_video(path: str | Path, frames: np.ndarray, fps: float) -> None:
    """``frames (T, H, W, 3)`` uint8 RGB -> an mp4 file (OpenCV's writer; no GL, no ffmpeg binary)."""
    import cv2
    frames = np.asarray(frames)
    h, w = frames.shape[1:3]
    wr = cv2.VideoWriter(str(path), cv2.VideoWriter_fourcc(*"mp4v"), float(fps), (w, h))
    if not wr.isOpened():
        raise OSError(f"cannot open a video writer for {path}")
    try:
        for f in frames:
            wr.write(cv2.cvtColor(np.ascontiguousarray(f[..., :3], dtype=np.uint8), cv2.COLOR_RGB2BGR))
    finally:
        wr.release()


def create_grid_summary_video(video_paths: list[str], success_statuses: list[bool], output_path: str | Path,
                              fps: float, highlight_duration: float = 1.0, grid_size: tuple[int, int] | None = None,
                              frame_stride: int = 1, border: int = 6) -> None:
    """Tiles the per-episode clips into one video.  Clips are read one frame at a time (memory: one frame per clip
    plus the grid); a clip that ends early keeps showing its last frame; every ``frame_stride``-th composed frame is
    written; the final composed frame is held for ``highlight_duration`` seconds with a green (success) or red
    (failure) border around each tile."""
    import cv2
    if len(video_paths) != len(success_statuses):
        raise ValueError(f"{len(video_paths)} videos but {len(success_statuses)} success flags")
    pairs = [(p, s) for p, s in zip(video_paths, success_statuses) if Path(p).exists()]
    if not pairs:
        logging.error("no episode clips found: no grid summary written")
        return
    n = len(video_paths)
    if grid_size is None:
        rows = int(np.ceil(np.sqrt(n)))
        grid_size = (rows, int(np.ceil(n / rows)))
    rows, cols = grid_size
    if n > rows * cols:
        raise ValueError(f"{n} videos do not fit a {rows} x {cols} grid")
    caps = [cv2.VideoCapture(p) for p, _ in pairs]
    wr = None
    try:
        ok, first = caps[0].read()
        if not ok:
            raise OSError(f"cannot decode {pairs[0][0]}")
        fh, fw = first.shape[:2]
        last: list[np.ndarray | None] = [first] + [None] * (len(caps) - 1)
        live = [True] * len(caps)
        wr = cv2.VideoWriter(str(output_path), cv2.VideoWriter_fourcc(*"mp4v"), float(fps), (fw * cols, fh * rows))
        if not wr.isOpened():
            raise OSError(f"cannot open a video writer for {output_path}")

        def compose() -> np.ndarray:
            grid = np.zeros((fh * rows, fw * cols, 3), np.uint8)
            for i, f in enumerate(last):
                if f is not None and f.shape[:2] == (fh, fw):
                    r, c = divmod(i, cols)
                    grid[r * fh:(r + 1) * fh, c * fw:(c + 1) * fw] = f
            return grid

        idx, grid, first_round = 0, None, True
        while True:
            advanced = first_round
            for i, cap in enumerate(caps):
                if not live[i] or (first_round and i == 0):
                    continue
                ok, f = cap.read()
                if ok:
                    last[i], advanced = f, True
                else:
                    live[i] = False
            first_round = False
            if not advanced:
                break
            grid = compose()
            if idx % max(1, frame_stride) == 0:
                wr.write(grid)
            idx += 1
        if grid is not None:
            for i, (_, ok_) in enumerate(pairs):
                r, c = divmod(i, cols)
                color = (0, 200, 0) if ok_ else (0, 0, 220)          # BGR
                cv2.rectangle(grid, (c * fw, r * fh), ((c + 1) * fw - 1, (r + 1) * fh - 1), color, border)
            for _ in range(max(1, int(round(highlight_duration * fps)))):
                wr.write(grid)
    finally:
        for cap in caps:
            cap.release()
        if wr is not None:
            wr.release()


def eval_policy(env, policy, n_episodes: int, start_seed: int | None = None, cfg=None, device=None,
                seed_list: list[int] | None = None, max_episodes_rendered: int = 0, videos_dir: Path | None = None,
                grid_size: tuple[int, int] | None = None, goal_frames_dir: Path | str | None = None,
                task_name: str = "task", rank: int = 0, keep_per_episode_videos: bool = False,
                video_frame_stride: int = 1, subgoal_generator=None) -> dict[str, Any]:
    """Collects ``n_episodes`` episodes; only steps up to (and including) the first ``done`` count.

    ``max_episodes_rendered > 0`` writes ``videos_dir/eval_episode_<i>.mp4`` for the first episodes and tiles them
    into ``videos_dir/grid_summary.mp4`` (the clips are removed afterwards unless ``keep_per_episode_videos``).
    ``goal_frames_dir`` saves the final camera frames of every SUCCESSFUL episode as
    ``<task>__seed<seed>__<camera>__rank<r>.png`` and lists them under ``goal_frames`` in the result, so a scene
    that one checkpoint fails can later be filled in from a checkpoint that solves the same seed."""
    import threading
    t0 = time.time()
    policy.eval()
    if max_episodes_rendered > 0 and videos_dir is None:
        raise ValueError("max_episodes_rendered > 0 needs videos_dir")
    n_batches = -(-n_episodes // env.num_envs)
    sum_r, max_r, succ, seeds_used = [], [], [], []
    accel_streams: list[list[float]] = []
    accel_provenance = None
    goal_rows: list[dict] = []
    video_paths: list[str] = []
    rendered_ok: list[bool] = []
    threads: list = []
    fps = float(getattr(getattr(env, "envs", [None])[0], "metadata", {}).get("render_fps", 30)) \
        if getattr(env, "envs", None) else 30.0
    if goal_frames_dir is not None:
        goal_frames_dir = Path(goal_frames_dir)
        goal_frames_dir.mkdir(parents=True, exist_ok=True)
    for b in range(n_batches):
        ep_frames: list[np.ndarray] = []
        n_now = max(0, min(max_episodes_rendered - len(video_paths), env.num_envs))

        def render_frame(e, _n=n_now, _dst=ep_frames):
            if _n > 0:
                _dst.append(np.stack([np.asarray(f) for f in e.call("render")[:_n]]))
        if seed_list is not None:
            seeds = list(seed_list[b * env.num_envs:(b + 1) * env.num_envs])
            seeds += [seeds[-1] + i + 1 for i in range(env.num_envs - len(seeds))]
        elif start_seed is not None:
            seeds = list(range(start_seed + b * env.num_envs, start_seed + (b + 1) * env.num_envs))
        else:
            seeds = None
        data = rollout(env, policy, seeds, cfg, device, subgoal_generator=subgoal_generator,
                       render_callback=render_frame if n_now > 0 else None,
                       capture_last_frames=goal_frames_dir is not None)
        T = data["done"].shape[1]
        first_done = torch.argmax(data["done"].to(torch.int), dim=1)
        first_done[~data["done"].any(dim=1)] = T - 1
        mask = (torch.arange(T)[None, :] <= first_done[:, None]).float()
        sum_r += (data["reward"] * mask).sum(1).tolist()
        max_r += torch.where(mask.bool(), data["reward"], torch.full_like(data["reward"], -float("inf"))).max(1).values.tolist()
        batch_succ = ((data["success"].float() * mask).sum(1) > 0).tolist()
        succ += batch_succ
        seeds_used += seeds if seeds is not None else [None] * env.num_envs
        if "accel" in data:
            accel_streams += data["accel"]
            accel_provenance = accel_provenance or data.get("accel_provenance")
        n_real = max(0, min(env.num_envs, n_episodes - b * env.num_envs))      # the last batch may overshoot
        if goal_frames_dir is not None and seeds is not None:
            import cv2
            for i in range(n_real):
                frames = data["last_frames"][i]
                if not batch_succ[i] or not frames:
                    continue
                row = {"task": task_name, "seed": int(seeds[i]), "success": 1}
                for cam, frame in sorted(frames.items()):
                    name = f"{task_name}__seed{int(seeds[i])}__{cam}__rank{rank}.png"
                    cv2.imwrite(str(goal_frames_dir / name), cv2.cvtColor(np.asarray(frame, np.uint8), cv2.COLOR_RGB2BGR))
                    row[cam] = name
                goal_rows.append(row)
        if ep_frames:
            stacked = np.stack(ep_frames, axis=1)                             # (n_now, T + 1, H, W, C)
            videos_dir = Path(videos_dir)
            videos_dir.mkdir(parents=True, exist_ok=True)
            for i in range(min(n_now, n_real)):
                path = videos_dir / f"eval_episode_{len(video_paths)}.mp4"
                video_paths.append(str(path))
                rendered_ok.append(bool(batch_succ[i]))
                th = threading.Thread(target=write_video, args=(path, stacked[i, :int(first_done[i]) + 2], fps))
                th.start()
                threads.append(th)
    for th in threads:
        th.join()
    extra: dict[str, Any] = {}
    if video_paths:
        grid = Path(videos_dir) / "grid_summary.mp4"
        try:
            create_grid_summary_video(video_paths, rendered_ok, grid, fps, highlight_duration=2.0, grid_size=grid_size,
                                      frame_stride=video_frame_stride)
            extra["video_paths"] = [str(grid)] + (video_paths if keep_per_episode_videos else [])
            if not keep_per_episode_videos:
                for p in video_paths:
                    Path(p).unlink(missing_ok=True)
        except Exception as exc:                              # a failed summary must not lose the evaluation
            logging.error("grid summary video failed: %s", exc)
            extra["video_paths"] = video_paths
    if accel_streams:
        extra["accel"] = {"streams": accel_streams[:n_episodes], "provenance": accel_provenance}
    if goal_frames_dir is not None:
        extra["goal_frames"] = goal_rows
        with open(goal_frames_dir / f"manifest_rank{rank}.jsonl", "a") as f:
            for row in goal_rows:
                f.write(json.dumps(row) + "\n")
    sum_r, max_r, succ, seeds_used = (x[:n_episodes] for x in (sum_r, max_r, succ, seeds_used))
    dt = time.time() - t0
    return {
        **extra,
        "per_episode": [{"episode_ix": i, "sum_reward": r, "max_reward": m, "success": bool(s), "seed": sd}
                        for i, (r, m, s, sd) in enumerate(zip(sum_r, max_r, succ, seeds_used))],
        "aggregated": {"avg_sum_reward": float(np.mean(sum_r)), "avg_max_reward": float(np.mean(max_r)),
                       "pc_success": float(np.mean(succ) * 100), "eval_s": dt, "eval_ep_s": dt / max(1, n_episodes)},
    }


def eval_policy_all(envs: dict[str, dict[int, Any]], policy, n_episodes: int, start_seed: int | None = None, cfg=None,
                    device=None, rank: int = 0, world: int = 1, seed_list: list[int] | None = None,
                    render: dict[str, Any] | None = None) -> dict[str, Any]:
    """Every (group, task) pair goes to rank ``index % world``; results are keyed ``group/task_id``.  ``render``:
    the video / goal-frame keyword arguments of :func:`eval_policy` (``videos_dir`` gets one sub-folder per task)."""
    tasks = [(g, tid, env) for g, by_id in envs.items() for tid, env in by_id.items()]
    mine: dict[str, Any] = {}
    for i, (g, tid, env) in enumerate(tasks):
        if i % world != rank:
            continue
        kw = dict(render or {})
        if kw.get("videos_dir") is not None:
            kw["videos_dir"] = Path(kw["videos_dir"]) / f"{g}_{tid}"
        mine[f"{g}/{tid}"] = eval_policy(env, policy, n_episodes, start_seed, cfg, device, seed_list,
                                         task_name=f"{g}_{tid}", rank=rank, **kw)
    return mine


def consolidate_eval_info(per_rank: list[dict[str, Any]]) -> dict[str, Any]:
    """Merges the per-rank ``{group/task: result}`` dicts: per-task, per-group and overall aggregates."""
    merged: dict[str, Any] = {}
    for d in per_rank:
        merged.update(d)
    per_group: dict[str, list[dict]] = {}
    for key, res in merged.items():
        per_group.setdefault(key.split("/")[0], []).extend(res["per_episode"])

    def agg(eps: list[dict]) -> dict[str, float]:
        if not eps:
            return {"avg_sum_reward": float("nan"), "avg_max_reward": float("nan"), "pc_success": float("nan"), "n": 0}
        return {"avg_sum_reward": float(np.mean([e["sum_reward"] for e in eps])),
                "avg_max_reward": float(np.mean([e["max_reward"] for e in eps])),
                "pc_success": float(np.mean([e["success"] for e in eps]) * 100), "n": len(eps)}

    every = [e for eps in per_group.values() for e in eps]
    info = {"per_task": {k: v["aggregated"] for k, v in merged.items()},
            "per_group": {g: agg(eps) for g, eps in per_group.items()}, "aggregated": agg(every),
            "per_episode": {k: v["per_episode"] for k, v in merged.items()}}
    # per-task accel streams (index-aligned with per_episode) and their provenance: what the calibration tool reads
    accel = {k: v["accel"] for k, v in merged.items() if v.get("accel")}
    if accel:
        info["accel"] = accel
    return info


def eval_policy_on_config(policy, cfg: TrainPipelineConfig, device, rank: int = 0, world: int = 1,
                          videos_dir: Path | None = None) -> dict[str, Any]:
    """Fresh environments, evaluate, gather, close: what the trainer calls every ``eval_freq`` steps.  With
    ``videos_dir`` the first ``eval.max_episodes_rendered`` episodes of every task are rendered into a grid video;
    ``eval.goal_frames_dir`` switches the goal-frame harvest on."""
    env_cfg = resolve_env_config(cfg.env)
    ev = cfg.eval
    render: dict[str, Any] = {}
    if videos_dir is not None and ev.max_episodes_rendered > 0:
        render.update(max_episodes_rendered=ev.max_episodes_rendered, videos_dir=videos_dir, grid_size=ev.grid_size,
                      keep_per_episode_videos=ev.keep_per_episode_videos, video_frame_stride=ev.video_frame_stride)
    if ev.goal_frames_dir:
        render["goal_frames_dir"] = ev.goal_frames_dir
    envs = make_envs(env_cfg, n_envs=ev.batch_size, use_async_envs=ev.use_async_envs)
    was_training = policy.training
    try:
        base = ev.seed if ev.seed is not None else cfg.seed          # the pipeline seed is the fallback
        n_tasks = sum(len(by_id) for by_id in envs.values())
        n_batches = -(-ev.n_episodes // max(1, ev.batch_size))
        span = max(1, n_batches * ev.batch_size * max(1, n_tasks))          # seeds one rank can consume
        seed = None if base is None else base + _rank_seed_offset(rank, ev.decorrelate_rank_seeds, span)
        mine = eval_policy_all(envs, policy, ev.n_episodes, seed, cfg, device, rank, world, ev.seed_list,
                               render or None)
    finally:
        close_envs(envs)
        policy.train(was_training)
    return consolidate_eval_info(control.gather_object(mine))


@parser.wrap()
def eval_main(cfg: TrainPipelineConfig):
    from ..policies.factory import make_policy
    from ..utils.logging_utils import init_logging
    from ..utils.random_utils import set_seed
    from .train import init_distributed
    rank, world, device = init_distributed()
    init_logging(rank)
    if cfg.env is None:
        raise ValueError("an `env` block is required for evaluation")
    if cfg.policy is None or not cfg.policy.pretrained_path:
        logging.warning("no pretrained policy path given: evaluating randomly initialised weights")
    if cfg.seed is not None:
        set_seed(cfg.seed, rank)
    if cfg.policy is not None:
        validate_eval_input_resolution(cfg)
    policy = make_policy(cfg.policy).to(device)
    if device.type == "cuda":
        policy.to(torch.bfloat16)
    policy.eval()
    from ..policies.accel import configure_accel
    from ..policies.candidates import configure_candidates
    if configure_accel(policy, cfg) is not None:               # cfg.policy.accel_prefix or $OPENTAU_ACCEL_PREFIX
        logging.info("accel streams are recorded per episode (prefix %d)", policy.accel_prefix)
    # best-of-N widens the expert batch by n_candidates per environment; a config that asks for it without naming a
    # critic is refused there rather than silently evaluated on a single sample
    configure_candidates(policy, cfg, device=device)
    out = Path(cfg.output_dir or "outputs/eval")
    info = eval_policy_on_config(policy, cfg, device, rank, world, videos_dir=out / "videos")
    if rank == 0:
        out.mkdir(parents=True, exist_ok=True)
        (out / "eval_info.json").write_text(json.dumps(info, indent=2))
        logging.info("success %.1f%% over %d episodes -> %s", info["aggregated"]["pc_success"],
                     info["aggregated"]["n"], out / "eval_info.json")
    return info


def main() -> None:
    eval_main()


if __name__ == "__main__":
    main()
