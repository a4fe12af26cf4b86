"""Smoke inference: N timed ``sample_actions`` calls on a dummy observation
(reference ``src/opentau/scripts/inference.py:44-136``)."""

from __future__ import annotations

import logging
import time

import torch

from ..configs import parser
from ..configs.train import TrainPipelineConfig
from ..policies.factory import make_policy
from ..utils.logging_utils import init_logging
from ..utils.utils import auto_torch_device, create_dummy_observation


@parser.wrap()
def inference_main(cfg: TrainPipelineConfig, n: int = 10):
    init_logging()
    device = auto_torch_device()
    policy = make_policy(cfg.policy).to(device)
    if device.type == "cuda":
        policy.to(torch.bfloat16)
    policy.eval()
    from ..policies.accel import configure_accel
    from ..policies.candidates import configure_candidates
    accel_prefix = configure_accel(policy, cfg)          # cfg.policy.accel_prefix or $OPENTAU_ACCEL_PREFIX
    n_candidates = configure_candidates(policy, cfg, device=device)   # before the first call: fails at start-up
    obs = create_dummy_observation(cfg, device)
    times = []
    with torch.inference_mode():
        for i in range(n):
            if device.type == "cuda":
                torch.cuda.synchronize()
            t0 = time.perf_counter()
            actions = policy.sample_actions(obs)
            if device.type == "cuda":
                torch.cuda.synchronize()
            times.append((time.perf_counter() - t0) * 1e3)
            logging.info("call %d: %.2f ms, actions %s%s", i, times[-1], tuple(actions.shape),
                         f", accel {policy.last_accel}" if accel_prefix else "")
    if n_candidates > 1:
        logging.info("best-of-%d: each call denoises %d candidates and a critic keeps one", n_candidates, n_candidates)
    logging.info("first %.2f ms; mean of the rest %.2f ms", times[0], sum(times[1:]) / max(1, len(times) - 1))
    return times


if __name__ == "__main__":
    inference_main()
