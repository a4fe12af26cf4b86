"""RECAP step 1 diagnostics: run a trained value model over episodes and dump value-vs-time curves
(reference ``src/opentau/scripts/calculate_value.py:66-285``).

Writes ``<output>/values.json`` = ``{episode: [{"frame": i, "value": v, "return": r_norm}, ...]}`` so that a
monotone climb towards 0 on successful episodes (and a drop towards ``C_neg / normalizer`` on failures) can be
checked by eye or by the bundled summary (Spearman correlation of value with time per episode).

    python -m opentau_b200.scripts.calculate_value --config_path=<value checkpoint> --episodes 0 1 2 --output out_dir
"""

from __future__ import annotations

import argparse
import json
import logging
from pathlib import Path

import numpy as np
import torch
from torch.utils.data import DataLoader, Subset

from ..configs import parser
from ..configs.train import TrainPipelineConfig
from ..datasets.dataset_mixture import collate_standard
from ..datasets.factory import make_dataset
from ..policies.factory import get_policy_class
from ..utils.logging_utils import init_logging
from ..utils.utils import auto_torch_device


def episode_values(policy, dataset, device, episodes: list[int] | None, batch_size: int = 16) -> dict[int, list[dict]]:
    idx = list(range(len(dataset)))
    if episodes is not None and hasattr(dataset, "episode_data_index"):
        idx = []
        for ep in episodes:
            i = dataset.epi2idx[ep]
            idx += list(range(int(dataset.episode_data_index["from"][i]), int(dataset.episode_data_index["to"][i])))
    out: dict[int, list[dict]] = {}
    loader = DataLoader(Subset(dataset, idx), batch_size=batch_size, shuffle=False, collate_fn=collate_standard)
    with torch.inference_mode():
        for batch in loader:
            batch = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
            vals = policy.predict_value(batch).float().cpu().tolist()
            for ep, fr, v, r in zip(batch["episode_index"], batch["frame_index"], vals, batch["return_continuous"]):
                out.setdefault(int(ep), []).append({"frame": int(fr), "value": float(v), "return": float(r)})
    return out


def summarize(curves: dict[int, list[dict]]) -> dict[int, dict[str, float]]:
    from scipy.stats import spearmanr
    res = {}
    for ep, rows in curves.items():
        rows = sorted(rows, key=lambda r: r["frame"])
        v = np.array([r["value"] for r in rows])
        t = np.arange(len(v))
        rho = float(spearmanr(t, v).statistic) if len(v) > 2 and np.ptp(v) > 0 else 0.0
        res[ep] = {"frames": len(v), "first": float(v[0]), "last": float(v[-1]), "spearman_time": rho,
                   "l1_to_return": float(np.mean(np.abs(v - np.array([r["return"] for r in rows]))))}
    return res


def main() -> None:
    init_logging()
    ap = argparse.ArgumentParser(add_help=False)
    ap.add_argument("--episodes", type=int, nargs="*", default=None)
    ap.add_argument("--output", default="outputs/value_curves")
    ap.add_argument("--dataset", type=int, default=0, help="index into dataset_mixture.datasets")
    args, rest = ap.parse_known_args()
    cfg: TrainPipelineConfig = parser.parse_config(TrainPipelineConfig, rest)
    device = auto_torch_device()
    policy = get_policy_class(cfg.policy.type).from_pretrained(cfg.policy.pretrained_path, config=cfg.policy).to(device)
    if device.type == "cuda":
        policy.to(torch.bfloat16)
    policy.eval()
    res = make_dataset(cfg.dataset_mixture.datasets[args.dataset], cfg)
    ds = res[0] if isinstance(res, tuple) else res
    curves = episode_values(policy, ds, device, args.episodes, cfg.batch_size)
    out = Path(args.output)
    out.mkdir(parents=True, exist_ok=True)
    (out / "values.json").write_text(json.dumps({str(k): v for k, v in curves.items()}, indent=1))
    for ep, s in summarize(curves).items():
        logging.info("episode %d: %s", ep, s)


if __name__ == "__main__":
    main()
