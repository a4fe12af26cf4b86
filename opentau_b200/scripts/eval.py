"""``opentau-eval``: closed-loop rollouts of a policy in (vectorised) environments.

Pipeline and result schema follow the reference (``src/opentau/scripts/eval.py:85-1567``): ``rollout`` steps a vector
environment until every sub-environment finished once, ``eval_policy`` repeats rollouts until ``n_episodes`` are
collected and reports per-episode ``sum_reward / max_reward / success / seed`` and the aggregate
``avg_sum_reward / avg_max_reward / pc_success / eval_s / eval_ep_s``, ``eval_policy_all`` walks the task groups
with tasks dealt round-robin to the ranks, and ``consolidate_eval_info`` merges the per-rank results into
``eval_info.json``.  Rendering-based outputs (grid videos, goal-frame harvest) need a graphics stack and are left
out; the headless ``fake`` environment supplies pixels rendered on the CPU.
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
from ..configs.train import TrainPipelineConfig
from ..envs.configs import EnvConfig
from ..envs.factory import make_envs
from ..envs.utils import add_envs_task, add_subgoal_images, check_env_attributes_and_types, preprocess_observation
from ..parallel import control


def resolve_env_config(env: Any) -> EnvConfig:
    if isinstance(env, EnvConfig):
        return env
    if isinstance(env, dict):
        d = dict(env)
        return EnvConfig.get_choice_class(d.pop("type"))(**d)
    raise TypeError(f"cannot build an environment from {type(env).__name__}")


def _rank_seed_offset(rank: int, decorrelate: bool) -> int:
    """Ranks evaluate different seeds unless asked to repeat the same ones."""
    return rank * 100_003 if decorrelate else 0


def rollout(env, policy, seeds: list[int] | None = None, cfg=None, device=None, return_observations: bool = False,
            extra_batch: dict[str, Any] | None = None, subgoal_generator=None) -> dict[str, Tensor]:
    """One batch of episodes.  Returns ``action (B,T,A)``, ``reward (B,T)``, ``success (B,T)``, ``done (B,T)``.
    ``subgoal_generator`` (``envs.subgoal``) pins one subgoal per sub-environment at the reset and feeds it to the
    policy at every step."""
    device = device or next(policy.parameters()).device
    policy.reset()
    obs, _ = env.reset(seed=seeds)
    check_env_attributes_and_types(env)
    if subgoal_generator is not None:
        subgoal_generator.start_episode(list(add_envs_task(env, preprocess_observation(obs, cfg))["prompt"]), seeds)
    max_steps = int(env.call("_max_episode_steps")[0])
    done = np.zeros(env.num_envs, dtype=bool)
    all_a, all_r, all_s, all_d, all_o = [], [], [], [], []
    step = 0
    while not done.all() and step < max_steps:
        batch = preprocess_observation(obs, cfg)
        batch = add_envs_task(env, batch)
        batch = add_subgoal_images(batch, subgoal_generator)
        batch = {k: (v.to(device) if isinstance(v, Tensor) else v) for k, v in batch.items()}
        if extra_batch:
            batch.update(extra_batch)
        if return_observations:
            all_o.append({k: v.cpu() for k, v in batch.items() if isinstance(v, Tensor)})
        with torch.inference_mode():
            action = policy.select_action(batch)
        a = action.float().cpu().numpy()
        obs, reward, terminated, truncated, info = env.step(a)
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
    return out


def eval_policy(env, policy, n_episodes: int, start_seed: int | None = None, cfg=None, device=None,
                seed_list: list[int] | None = None) -> dict[str, Any]:
    """Collects ``n_episodes`` episodes; only steps up to (and including) the first ``done`` count."""
    t0 = time.time()
    policy.eval()
    n_batches = -(-n_episodes // env.num_envs)
    sum_r, max_r, succ, seeds_used = [], [], [], []
    for b in range(n_batches):
        if seed_list is not None:
            seeds = list(seed_list[b * env.num_envs:(b + 1) * env.num_envs])
            seeds += [seeds[-1] + i + 1 for i in range(env.num_envs - len(seeds))]
        elif start_seed is not None:
            seeds = list(range(start_seed + b * env.num_envs, start_seed + (b + 1) * env.num_envs))
        else:
            seeds = None
        data = rollout(env, policy, seeds, cfg, device)
        T = data["done"].shape[1]
        first_done = torch.argmax(data["done"].to(torch.int), dim=1)
        first_done[~data["done"].any(dim=1)] = T - 1
        mask = (torch.arange(T)[None, :] <= first_done[:, None]).float()
        sum_r += (data["reward"] * mask).sum(1).tolist()
        max_r += torch.where(mask.bool(), data["reward"], torch.full_like(data["reward"], -float("inf"))).max(1).values.tolist()
        succ += ((data["success"].float() * mask).sum(1) > 0).tolist()
        seeds_used += seeds if seeds is not None else [None] * env.num_envs
    sum_r, max_r, succ, seeds_used = (x[:n_episodes] for x in (sum_r, max_r, succ, seeds_used))
    dt = time.time() - t0
    return {
        "per_episode": [{"episode_ix": i, "sum_reward": r, "max_reward": m, "success": bool(s), "seed": sd}
                        for i, (r, m, s, sd) in enumerate(zip(sum_r, max_r, succ, seeds_used))],
        "aggregated": {"avg_sum_reward": float(np.mean(sum_r)), "avg_max_reward": float(np.mean(max_r)),
                       "pc_success": float(np.mean(succ) * 100), "eval_s": dt, "eval_ep_s": dt / max(1, n_episodes)},
    }


def eval_policy_all(envs: dict[str, dict[int, Any]], policy, n_episodes: int, start_seed: int | None = None, cfg=None,
                    device=None, rank: int = 0, world: int = 1, seed_list: list[int] | None = None) -> dict[str, Any]:
    """Every (group, task) pair goes to rank ``index % world``; results are keyed ``group/task_id``."""
    tasks = [(g, tid, env) for g, by_id in envs.items() for tid, env in by_id.items()]
    mine: dict[str, Any] = {}
    for i, (g, tid, env) in enumerate(tasks):
        if i % world != rank:
            continue
        mine[f"{g}/{tid}"] = eval_policy(env, policy, n_episodes, start_seed, cfg, device, seed_list)
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
    return {"per_task": {k: v["aggregated"] for k, v in merged.items()},
            "per_group": {g: agg(eps) for g, eps in per_group.items()}, "aggregated": agg(every),
            "per_episode": {k: v["per_episode"] for k, v in merged.items()}}


def eval_policy_on_config(policy, cfg: TrainPipelineConfig, device, rank: int = 0, world: int = 1) -> dict[str, Any]:
    """Fresh environments, evaluate, gather, close: what the trainer calls every ``eval_freq`` steps."""
    env_cfg = resolve_env_config(cfg.env)
    ev = cfg.eval
    envs = make_envs(env_cfg, n_envs=ev.batch_size, use_async_envs=ev.use_async_envs)
    was_training = policy.training
    try:
        seed = None if ev.seed is None else ev.seed + _rank_seed_offset(rank, ev.decorrelate_rank_seeds)
        mine = eval_policy_all(envs, policy, ev.n_episodes, seed, cfg, device, rank, world, ev.seed_list)
    finally:
        for by_id in envs.values():
            for e in by_id.values():
                e.close()
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
    if getattr(cfg.policy, "n_candidates", 1) > 1 and not getattr(cfg.policy, "action_chunk_critic_path", None):
        logging.info("best-of-N without a critic: the medoid candidate is used")
    if cfg.seed is not None:
        set_seed(cfg.seed, rank)
    policy = make_policy(cfg.policy).to(device)
    if device.type == "cuda":
        policy.to(torch.bfloat16)
    policy.eval()
    info = eval_policy_on_config(policy, cfg, device, rank, world)
    if rank == 0:
        out = Path(cfg.output_dir or "outputs/eval")
        out.mkdir(parents=True, exist_ok=True)
        (out / "eval_info.json").write_text(json.dumps(info, indent=2))
        logging.info("success %.1f%% over %d episodes -> %s", info["aggregated"]["pc_success"],
                     info["aggregated"]["n"], out / "eval_info.json")
    return info


def main() -> None:
    eval_main()


if __name__ == "__main__":
    main()
