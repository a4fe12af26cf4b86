"""``opentau-accel-diagnose``: measure the numerical noise floor of the ``accel`` score on a checkpoint
(reference ``src/opentau/scripts/diagnose_accel.py``).

``accel`` is built from differences of nearly equal velocity predictions, so in bf16 there is a positive floor
beneath it.  This tool samples the same observation twice with the SAME noise (the difference of the two scores is
pure rounding / nondeterminism) and with different noise (the spread the detector sees), in the serving dtype and
in fp32, and reports the ratio: a calibration whose successful-rollout scores sit within a small multiple of the
floor measures rounding, not geometry.

    opentau-accel-diagnose --config_path=<checkpoint> --samples 16
"""

from __future__ import annotations

import argparse
import json
import logging

import torch

from ..configs import parser
from ..configs.train import TrainPipelineConfig
from ..policies.accel import configure_accel
from ..policies.factory import make_policy
from ..utils.utils import auto_torch_device, create_dummy_observation


@torch.no_grad()
def accel_samples(policy, obs, n: int, same_noise: bool, seed: int = 0) -> list[float]:
    cfg = policy.config
    out = []
    for i in range(n):
        g = torch.Generator(device="cpu").manual_seed(seed if same_noise else seed + i)
        noise = torch.randn(obs["state"].shape[0], cfg.chunk_size, cfg.max_action_dim, generator=g).to(obs["state"].device)
        policy.sample_actions(obs, noise=noise)
        acc = getattr(policy, "last_accel", None)
        out.append(float(acc[0]) if acc else float("nan"))
    return out


def diagnose(policy, cfg, device, samples: int = 8) -> dict:
    obs = create_dummy_observation(cfg, device)
    res = {}
    for name, dtype in (("serving", torch.bfloat16 if device.type == "cuda" else torch.float32), ("fp32", torch.float32)):
        policy.to(dtype)
        same = torch.tensor(accel_samples(policy, obs, samples, same_noise=True))
        diff = torch.tensor(accel_samples(policy, obs, samples, same_noise=False))
        res[name] = {"mean": float(diff.nanmean()), "spread_across_noise": float(diff[~diff.isnan()].std()) if samples > 1 else 0.0,
                     "repeatability_floor": float((same - same[0]).abs().max()), "n": samples}
    f = res["serving"]["repeatability_floor"]
    res["spread_over_floor"] = res["serving"]["spread_across_noise"] / f if f > 0 else float("inf")
    return res


def main() -> None:
    ap = argparse.ArgumentParser(add_help=False)
    ap.add_argument("--samples", type=int, default=8)
    ap.add_argument("--prefix", default="auto")
    args, rest = ap.parse_known_args()
    cfg: TrainPipelineConfig = parser.parse_config(TrainPipelineConfig, rest)
    device = auto_torch_device()
    policy = make_policy(cfg.policy).to(device).eval()
    configure_accel(policy, args.prefix)
    out = diagnose(policy, cfg, device, args.samples)
    logging.info("accel noise floor: %s", out)
    print(json.dumps(out, indent=2))


if __name__ == "__main__":
    main()
