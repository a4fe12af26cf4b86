"""``make_optimizer_and_scheduler(cfg, policy)`` for the generic (torch.optim) path
(reference ``src/opentau/optim/factory.py:26``)."""

from __future__ import annotations


def make_optimizer_and_scheduler(cfg, policy):
    params = policy.get_optim_params() if hasattr(policy, "get_optim_params") else policy.parameters()
    optimizer = cfg.optimizer.build(params)
    scheduler = cfg.scheduler.build(optimizer, cfg.steps) if cfg.scheduler is not None else None
    return optimizer, scheduler
