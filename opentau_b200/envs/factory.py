"""``make_envs(cfg, n_envs)`` -> ``{task_group: {task_id: vector_env}}`` (reference ``src/opentau/envs/factory.py:45-225``)."""

from __future__ import annotations

from .configs import EnvConfig, FakeEnvConfig
from .fake import FakeRobotEnv, SyncVectorEnv

UNAVAILABLE = ("{name} renders through MuJoCo on OpenGL/EGL, and no graphics stack exists on this machine; "
               "use `env.type=fake` to exercise the evaluation pipeline headlessly")


def make_env_config(env_type: str, **kwargs) -> EnvConfig:
    return EnvConfig.get_choice_class(env_type)(**kwargs)


def make_envs(cfg: EnvConfig, n_envs: int = 1, use_async_envs: bool = False) -> dict[str, dict[int, SyncVectorEnv]]:
    if n_envs < 1:
        raise ValueError("`n_envs` must be at least 1")
    if isinstance(cfg, FakeEnvConfig):
        groups = cfg.task_groups or {cfg.task or "fake": list(range(len(cfg.tasks)))}
        out: dict[str, dict[int, SyncVectorEnv]] = {}
        for g, ids in groups.items():
            out[g] = {}
            for tid in ids:
                def fn(tid=tid):
                    return FakeRobotEnv(cfg.tasks[tid % len(cfg.tasks)], cfg.state_dim, cfg.action_dim, cfg.num_cams,
                                        cfg.resolution, cfg.tolerance, cfg.action_scale, cfg.episode_length, tid)
                out[g][tid] = SyncVectorEnv([fn] * n_envs)
        return out
    try:
        if cfg.type == "libero":
            from .libero import create_libero_envs
            return create_libero_envs(cfg, n_envs)
        if cfg.type == "robocasa":
            from .robocasa import create_robocasa_envs
            return create_robocasa_envs(cfg, n_envs)
    except ImportError as e:
        raise RuntimeError(UNAVAILABLE.format(name=cfg.type) + f" ({e})") from e
    raise RuntimeError(UNAVAILABLE.format(name=cfg.type))
