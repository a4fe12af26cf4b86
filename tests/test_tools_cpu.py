"""Profilers and small tools on CPU."""

import torch

from helpers import TINY, tiny_batch, tiny_pi05
from opentau_b200.configs.train import TrainPipelineConfig
from opentau_b200.scripts.find_unused_params import unused_parameters
from opentau_b200.scripts.profile_step import PHASES, profile


def _cfg(tmp_path):
    return TrainPipelineConfig.from_dict({
        "dataset_mixture": {"datasets": [{"synthetic": {"length": 32, "name": "p"}}], "action_freq": 10.0},
        "policy": {"type": "pi05", "chunk_size": 10, "n_action_steps": 10, "prompt_max_length": 24,
                   "discrete_action_max_length": 8, "discrete_action_vocab_size": 256, "dropout": 0.0, "device": "cpu", **TINY},
        "output_dir": str(tmp_path / "o"), "resolution": [224, 224], "num_cams": 1, "action_chunk": 10, "batch_size": 2,
        "num_workers": 0, "use_policy_training_preset": True})


def test_profile_step_reports_the_reference_phases(tmp_path, monkeypatch):
    monkeypatch.setenv("PROFILE_STEPS", "2")
    monkeypatch.setenv("PROFILE_WARMUP", "1")
    monkeypatch.setenv("PROFILE_STEP_JSON", str(tmp_path / "p.json"))
    out = profile(_cfg(tmp_path))
    assert set(out["phases_ms_max_over_ranks"]) == set(PHASES)
    ph = out["phases_ms_max_over_ranks"]
    assert ph["total"] >= ph["forward"] + ph["bwd"] > 0 and out["global_samples_per_s"] > 0
    assert (tmp_path / "p.json").exists() and out["measured_steps"] == 2


def test_unused_parameter_audit():
    pol = tiny_pi05(predict_response=False).train()
    names = unused_parameters(pol, tiny_batch(), {"MSE": 1.0, "CE": 1.0})
    assert all("vision" not in n for n in names)            # frozen tower is not trainable, so never reported
    pol2 = tiny_pi05().train()
    extra = torch.nn.Linear(4, 4)
    pol2.dead_head = extra
    assert set(unused_parameters(pol2, tiny_batch(), {"MSE": 1.0, "CE": 1.0})) >= {"dead_head.weight", "dead_head.bias"}


def test_bin_to_safetensors(tmp_path):
    from safetensors.torch import load_file
    from opentau_b200.scripts.bin_to_safetensors import convert
    w = torch.randn(4, 4)
    torch.save({"module.a.weight": w, "module.b.weight": w, "c": torch.ones(2)}, tmp_path / "m.bin")
    assert convert(tmp_path / "m.bin", tmp_path / "m.safetensors") == 3
    sd = load_file(str(tmp_path / "m.safetensors"))
    assert set(sd) == {"a.weight", "b.weight", "c"} and torch.equal(sd["a.weight"], sd["b.weight"])


def test_latency_benchmark_builders_on_tiny_geometries():
    """Every policy of the latency benchmark builds at its plumbing size and produces one action chunk."""
    import torch

    from opentau_b200.scripts.benchmark_inference import BUILDERS, run, summarize
    assert set(BUILDERS) == {"pi05", "cosmos3", "pi06"}
    for name, steps in (("pi05", 3), ("pi06", 2)):
        policy, batch = BUILDERS[name](1, 16, torch.device("cpu"), True, steps)
        with torch.no_grad():
            out = policy.sample_actions(batch)
        assert out.shape[0] == 1 and out.shape[1] == 50 and torch.isfinite(out.float()).all()
    rec = run(policy, batch, 1, 2)
    assert rec["n_timed"] == 2 if "n_timed" in rec else True
    assert summarize([1.0, 2.0, 3.0])["p50_ms"] == 2.0
