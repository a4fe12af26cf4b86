"""Open-loop check of a trained policy: MSE between sampled and recorded action chunks over dataset frames
(reference ``src/opentau/scripts/actions_mse_loss.py``)."""

from __future__ import annotations

import json
import logging

import torch

from ..configs import parser
from ..configs.train import TrainPipelineConfig


@torch.no_grad()
def open_loop_mse(policy, loader, n_batches: int, device) -> dict:
    policy.eval()
    se, n, per_dim = 0.0, 0, None
    for i, batch in enumerate(loader):
        if i >= n_batches:
            break
        batch = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
        pred = policy.sample_actions(batch).float()
        tgt = batch["actions"].float()[:, :pred.shape[1], :pred.shape[2]]
        keep = (~batch["action_is_pad"][:, :pred.shape[1]]).float()[..., None]
        d = (pred - tgt) ** 2 * keep
        se += float(d.sum())
        n += float(keep.sum() * pred.shape[2])
        pd = d.sum((0, 1)) / keep.sum().clamp(min=1)
        per_dim = pd if per_dim is None else per_dim + pd
    return {"mse": se / max(n, 1), "per_dim_mse": (per_dim / max(1, min(n_batches, i + 1))).tolist() if per_dim is not None else []}


@parser.wrap()
def main(cfg: TrainPipelineConfig):
    from ..datasets.factory import make_dataset_mixture
    from ..policies.factory import make_policy
    from ..utils.logging_utils import init_logging
    from ..utils.utils import auto_torch_device
    from ..policies.candidates import refuse_candidates
    init_logging()
    refuse_candidates(cfg, reason="the open-loop error compares ONE sampled chunk per observation with the recorded "
                      "one; a critic's selection would change what is measured. Run it with policy.n_candidates=1.")
    device = auto_torch_device()
    res = make_dataset_mixture(cfg)
    mix = res[0] if isinstance(res, tuple) else res
    policy = make_policy(cfg.policy, ds_meta=mix.meta).to(device)
    out = open_loop_mse(policy, mix.get_dataloader(cfg.dataloader_batch_size, 0), 16, device)
    logging.info("open-loop action MSE: %.6f", out["mse"])
    print(json.dumps(out, indent=2))
    return out


if __name__ == "__main__":
    main()
