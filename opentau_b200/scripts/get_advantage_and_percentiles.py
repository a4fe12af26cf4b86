"""RECAP step 2: advantages of every frame under a trained value model, and their percentiles
(reference ``src/opentau/scripts/get_advantage_and_percentiles.py:109-224``).

``A(t) = r_n(t) + V(t + N) - V(t)`` with the normalised n-step return ``r_n`` of ``policies/value/reward.py`` and
``V = 0`` past the end of an episode.  Writes ``meta/advantages.json`` (``"episode,timestamp" -> advantage``) into
each dataset root — the file :class:`LeRobotDatasetMetadata` reads back to emit the ``advantage`` key — and prints
the 0..100 % percentiles in steps of 5, from which the positive-advantage threshold of pi0 RECAP training is picked.

    python -m opentau_b200.scripts.get_advantage_and_percentiles --config_path=<value checkpoint> [--dataset_mixture=<json>]
"""

from __future__ import annotations

import json
import logging
import sys
from pathlib import Path

import numpy as np
import torch
from torch.utils.data import DataLoader

from ..configs import parser
from ..configs.default import DatasetMixtureConfig
from ..configs.train import TrainPipelineConfig
from ..datasets.dataset_mixture import collate_standard
from ..datasets.factory import make_dataset
from ..policies.factory import get_policy_class
from ..policies.value.reward import calculate_n_step_return
from ..utils.logging_utils import init_logging
from ..utils.random_utils import set_seed
from ..utils.utils import auto_torch_device

ADVANTAGES_PATH = "meta/advantages.json"


def _scalar(x):
    if isinstance(x, np.ndarray):
        x = torch.from_numpy(x)
    if isinstance(x, torch.Tensor):
        return x.item()
    return x


def compute_advantages(policy, dataset, cfg, device, batch_size: int, num_workers: int = 0) -> dict[tuple[int, float], float]:
    rc = cfg.policy.reward_config
    loader = DataLoader(dataset, batch_size=batch_size, shuffle=False, drop_last=False, num_workers=num_workers,
                        collate_fn=collate_standard)
    values: dict[tuple[int, int], tuple[float, float]] = {}
    frames: list[tuple[int, int, float]] = []
    with torch.inference_mode():
        for batch in loader:
            batch = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
            v0s = policy.predict_value(batch).float().cpu().tolist()
            for success, ep, end, cur, ts, v0 in zip(batch["success"], batch["episode_index"], batch["episode_end_idx"],
                                                     batch["current_idx"], batch["timestamp"], v0s):
                success, ep, end, cur, ts = bool(_scalar(success)), int(_scalar(ep)), int(_scalar(end)), int(_scalar(cur)), float(_scalar(ts))
                r = calculate_n_step_return(success, rc.N_steps_look_ahead, end, rc.reward_normalizer, cur, rc.C_neg)
                values[(ep, cur)] = (v0, r)
                frames.append((ep, cur, ts))
    out = {}
    for ep, cur, ts in frames:
        v0, r = values[(ep, cur)]
        vn = values.get((ep, cur + rc.N_steps_look_ahead), (0.0, 0.0))[0]
        out[(ep, ts)] = r + vn - v0
    return out


def _mixture_from_argv() -> tuple[str | None, list[str]]:
    path, rest = None, []
    for a in sys.argv[1:]:
        if a.startswith("--dataset_mixture_path=") or (a.startswith("--dataset_mixture=") and "." not in a.split("=", 1)[0]):
            path = a.split("=", 1)[1]
        else:
            rest.append(a)
    return path, rest


def main() -> None:
    init_logging()
    mix_path, argv = _mixture_from_argv()
    cfg: TrainPipelineConfig = parser.parse_config(TrainPipelineConfig, argv)
    if mix_path:
        from ..configs.codec import decode
        from ..configs.refs import load_json_with_refs as load_with_refs
        mix = decode(DatasetMixtureConfig, load_with_refs(mix_path))
    else:
        mix = cfg.dataset_mixture
    device = auto_torch_device()
    if cfg.seed is not None:
        set_seed(cfg.seed)
    policy = get_policy_class(cfg.policy.type).from_pretrained(cfg.policy.pretrained_path, config=cfg.policy).to(device)
    if device.type == "cuda":
        policy.to(torch.bfloat16)
    policy.eval()
    every: list[float] = []
    for i, dcfg in enumerate(mix.datasets):
        logging.info("dataset %d: %s", i, dcfg.name)
        res = make_dataset(dcfg, cfg, return_advantage_input=True)
        ds = res[0] if isinstance(res, tuple) else res
        adv = compute_advantages(policy, ds, cfg, device, cfg.batch_size, cfg.num_workers)
        every += list(adv.values())
        with open(Path(dcfg.root) / ADVANTAGES_PATH, "w") as f:
            json.dump({f"{ep},{ts}": f"{v:.6f}" for (ep, ts), v in adv.items()}, f, indent=4)
    pct = list(range(0, 101, 5))
    print("Advantage percentiles for deciding epsilon threshold:")
    for p, v in zip(pct, np.percentile(np.asarray(every), pct)):
        print(f"  {p:3d}th percentile: {v:.6f}")


if __name__ == "__main__":
    main()
