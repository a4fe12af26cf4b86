"""RECAP tooling on CPU: advantages A(t) = r_n + V(t+N) - V(t) written to meta/advantages.json and read back by the
dataset as the ``advantage`` key; value curves per episode."""

import json

import numpy as np
import torch

from helpers import TINY
from opentau_b200.configs.train import TrainPipelineConfig
from opentau_b200.datasets.factory import make_dataset
from opentau_b200.policies.factory import make_policy
from opentau_b200.scripts.calculate_value import episode_values, summarize
from opentau_b200.scripts.get_advantage_and_percentiles import ADVANTAGES_PATH, compute_advantages
from test_datasets_cpu import _record


def _cfg(root):
    return TrainPipelineConfig.from_dict({
        "dataset_mixture": {"datasets": [{"repo_id": "local/toy", "root": str(root)}], "action_freq": 10.0},
        "policy": {"type": "value", "prompt_max_length": 16, "response_max_length": 6, "device": "cpu",
                   "reward_config": {"number_of_bins": 21, "C_neg": -100.0, "reward_normalizer": 40, "N_steps_look_ahead": 3},
                   "vlm": dict(TINY["vlm"], sliding_window_pattern=2), "vision": TINY["vision"]},
        "resolution": [224, 224], "num_cams": 1, "action_chunk": 50, "batch_size": 8, "num_workers": 0})


class FixedValue(torch.nn.Module):
    """V(frame) = -(frames to go) / normaliser: the exact value of a success-only dataset."""

    def __init__(self, ends):
        super().__init__()
        self.ends = ends

    def predict_value(self, batch):
        return torch.tensor([-(int(e) - int(c) - 1) / 40.0 for e, c in zip(batch["episode_end_idx"], batch["current_idx"])])


def test_advantages_are_zero_under_the_true_value_function(tmp_path):
    _record(tmp_path / "toy", episodes=(6, 5))
    cfg = _cfg(tmp_path / "toy")
    ds = make_dataset(cfg.dataset_mixture.datasets[0], cfg, return_advantage_input=True)
    s = ds[2]
    assert s["success"] is True and s["episode_end_idx"] == 6 and s["current_idx"] == 2 and s["last_step"] is False
    assert s["return_bin_idx"].item() == int((-3 / 40 + 1) * 20) and abs(float(s["return_continuous"]) + 3 / 40) < 1e-6
    adv = compute_advantages(FixedValue(None), ds, cfg, "cpu", batch_size=4)
    assert len(adv) == 11 and max(abs(v) for v in adv.values()) < 1e-6
    (tmp_path / "toy" / ADVANTAGES_PATH).write_text(json.dumps({f"{ep},{ts}": "0.250000" for (ep, ts) in adv}))
    ds2 = make_dataset(cfg.dataset_mixture.datasets[0], cfg)
    assert float(ds2[3]["advantage"]) == 0.25


def test_value_curves_with_a_real_value_model(tmp_path):
    _record(tmp_path / "toy", episodes=(4, 4))
    cfg = _cfg(tmp_path / "toy")
    ds = make_dataset(cfg.dataset_mixture.datasets[0], cfg)
    from opentau_b200.datasets.dataset_mixture import DatasetMixtureMetadata
    pol = make_policy(cfg.policy, ds_meta=DatasetMixtureMetadata([ds], ["local/toy"], ["local/toy"])).eval()
    curves = episode_values(pol, ds, "cpu", episodes=[1], batch_size=4)
    assert set(curves) == {1} and [r["frame"] for r in sorted(curves[1], key=lambda r: r["frame"])] == [0, 1, 2, 3]
    s = summarize(curves)[1]
    assert s["frames"] == 4 and -1.0 <= s["first"] <= 0.0 and np.isfinite(s["l1_to_return"])
