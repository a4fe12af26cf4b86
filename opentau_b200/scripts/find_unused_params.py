"""Lists trainable parameters that receive no gradient from one forward/backward
(reference ``src/opentau/scripts/find_unused_params.py:88-184``).  The engine reduces one flat gradient buffer, so
unused parameters cost nothing at run time here; the audit is still useful to spot dead heads in a config."""

from __future__ import annotations

import logging

import torch

from ..configs import parser
from ..configs.train import TrainPipelineConfig
from ..datasets.factory import make_dataset_mixture
from ..parallel.engine import assemble_weighted_loss
from ..policies.factory import make_policy
from ..utils.logging_utils import init_logging


def unused_parameters(policy, batch, loss_weights) -> list[str]:
    for p in policy.parameters():
        p.grad = None
        if hasattr(p, "main_grad"):
            p.main_grad.zero_()
    loss = assemble_weighted_loss(policy(batch), loss_weights)
    loss.backward()
    out = []
    for name, p in policy.named_parameters():
        if not p.requires_grad:
            continue
        mg = getattr(p, "main_grad", None)
        touched = (p.grad is not None) or (mg is not None and bool(mg.abs().sum() > 0))
        if not touched:
            out.append(name)
    return out


@parser.wrap()
def find(cfg: TrainPipelineConfig) -> list[str]:
    init_logging()
    cfg.validate()
    res = make_dataset_mixture(cfg)
    mix = res[0] if isinstance(res, tuple) else res
    device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    policy = make_policy(cfg.policy, ds_meta=mix.meta).to(device).train()
    batch = next(iter(mix.get_dataloader(cfg.dataloader_batch_size, 0)))
    batch = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
    names = unused_parameters(policy, batch, cfg.loss_weighting)
    logging.info("%d trainable parameter tensors received no gradient", len(names))
    for n in names:
        logging.info("  %s", n)
    return names


if __name__ == "__main__":
    find()
