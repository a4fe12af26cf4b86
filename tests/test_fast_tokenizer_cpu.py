"""DCT + BPE action tokenizer: merges compress smooth trajectories, decoding inverts encoding up to quantisation."""

import numpy as np

from opentau_b200.scripts.fit_fast_tokenizer import fit
from opentau_b200.utils.tokenizer import BpeDctActionTokenizer


def _chunks(n=200, T=20, D=4, seed=0):
    rng = np.random.default_rng(seed)
    t = np.linspace(0, 1, T)[None, :, None]
    return rng.uniform(-1, 1, (n, 1, D)) + rng.uniform(-1, 1, (n, 1, D)) * t + 0.3 * np.sin(2 * np.pi * t * rng.integers(1, 3, (n, 1, D)))


def test_fit_compress_and_roundtrip(tmp_path):
    tok, rep = fit(np.clip(_chunks() / 2.5, -1, 1), vocab_size=512, max_token_length=64)
    assert rep["merges"] > 0 and rep["tokens_per_chunk_mean"] < rep["symbols_per_chunk_mean"]
    assert rep["reconstruction_rmse"] < 0.05 and 0.0 <= rep["share_above_max_token_length"] <= 1.0
    assert rep["tokens_per_chunk_percentiles"]["p50"] <= rep["tokens_per_chunk_percentiles"]["p100"]
    x = np.clip(_chunks(5, seed=7) / 2.5, -1, 1)
    ids = tok(x)
    assert all(0 < i < tok.vocab_size for row in ids for i in row)
    rec = tok.decode(ids)
    assert np.abs(rec - x).max() < 0.15
    tok.save(tmp_path / "t.json")
    again = BpeDctActionTokenizer.load(tmp_path / "t.json")
    assert again(x) == ids and again.vocab_size == tok.vocab_size


def test_native_trainer_and_encoder_match_the_reference_loops():
    import pytest
    from opentau_b200.utils.tokenizer import _bpe_lib
    if _bpe_lib() is None:
        pytest.skip("native byte-pair library not built")
    for seed, shape, vocab in ((0, (120, 20, 4), 500), (1, (40, 12, 3), 300), (2, (15, 8, 2), 260)):
        x = np.clip(_chunks(*shape, seed=seed) / 2.5, -1, 1)
        py = BpeDctActionTokenizer(scale=10.0).fit(x, vocab_size=vocab, native=False)
        nat = BpeDctActionTokenizer(scale=10.0).fit(x, vocab_size=vocab, native=True)
        assert py.merges == nat.merges and len(py.merges) > 0
        y = np.clip(_chunks(30, *shape[1:], seed=seed + 10) / 2.5, -1, 1)
        assert py(y, native=False) == py(y, native=True)
    # runs of one symbol: overlapping occurrences merge left to right ("a a a" -> "N a")
    flat = np.zeros((20, 16, 4))
    flat[:, :8] = 0.3
    py = BpeDctActionTokenizer(scale=10.0).fit(flat, vocab_size=300, native=False)
    nat = BpeDctActionTokenizer(scale=10.0).fit(flat, vocab_size=300, native=True)
    assert py.merges == nat.merges and py(flat, native=False) == nat(flat, native=True)
    assert BpeDctActionTokenizer()(np.zeros((2, 4, 2)), native=True) == [[], []]          # all-zero chunks: no symbols


def _toy_dataset(root, robot, shift, episodes=(14, 11)):
    from opentau_b200.datasets.lerobot_dataset import LeRobotDataset
    feats = {"observation.state": {"dtype": "float32", "shape": (3,), "names": None},
             "action": {"dtype": "float32", "shape": (3,), "names": None}}
    rec = LeRobotDataset.create(f"local/{robot}", fps=10, root=root, robot_type=robot, features=feats, use_videos=False)
    k = 0
    for e, n in enumerate(episodes):
        for t in range(n):
            s = np.array([np.sin(0.3 * k), np.cos(0.2 * k), 0.1 * t], np.float32) + shift
            rec.add_frame({"observation.state": s, "action": s + np.array([0.05, -0.05, 0.0], np.float32), "task": f"task {e}"})
            k += 1
        rec.save_episode()
    return rec


def test_fit_script_uses_the_policy_normalisation_per_head(tmp_path):
    import json
    from opentau_b200.scripts import fit_fast_tokenizer as fft
    from opentau_b200.utils.tokenizer import load_action_tokenizer
    _toy_dataset(tmp_path / "a", "arm", 0.0)
    _toy_dataset(tmp_path / "b", "rover", 10.0)
    mix = {"datasets": [{"repo_id": "local/arm", "root": str(tmp_path / "a"), "control_mode": "joint"},
                        {"repo_id": "local/rover", "root": str(tmp_path / "b"), "control_mode": "joint"}],
           "weights": [3.0, 1.0], "action_freq": 10.0}
    (tmp_path / "mix.json").write_text(json.dumps(mix))
    argv = ["--mixture-json", str(tmp_path / "mix.json"), "--out-dir", str(tmp_path / "tok"), "--chunk-size", "6",
            "--action-dim", "8", "--max-state-dim", "8", "--total-chunks", "200", "--vocab-size", "300"]
    rep = fft.run(fft.parse_args(argv))
    assert rep["per_dataset_chunks"] == [150, 50] and rep["n_norm_heads"] == 2
    assert rep["per_dataset_norm_keys"] == ["arm::joint", "rover::joint"]
    # each head is spread over its own range: the shifted dataset does not squeeze the other into a corner
    assert -1.001 <= rep["normalised_range"][0] and rep["normalised_range"][1] <= 1.001
    assert rep["roundtrip"]["merges"] > 0 and rep["roundtrip"]["reconstruction_rmse"] < 0.08
    assert "share_above_max_token_length" in rep["roundtrip"]
    side = json.loads((tmp_path / "tok" / "opentau_action_norm.json").read_text())
    assert side == {"config_version": fft.CURRENT_CONFIG_VERSION, "zero_range_center": fft.CURRENT_CONFIG_VERSION >= 1}
    tok = load_action_tokenizer(str(tmp_path / "tok"), vocab_size=2048)
    assert isinstance(tok, BpeDctActionTokenizer) and tok.action_dim == 8 and tok.time_horizon == 6
    import pytest
    with pytest.raises(ValueError, match="discrete_action_vocab_size"):
        load_action_tokenizer(str(tmp_path / "tok"), vocab_size=100)
    # the legacy pooled range under-spreads both heads
    glob = fft.run(fft.parse_args(argv + ["--no-per-head-norm", "--skip-fit", "--pilot"]))
    assert glob["normalization"] == "global" and glob["pilot"] and (tmp_path / "tok" / "pilot" / "fit_report.json").exists()
    assert fft.compute_budgets([1, 1, 1], 10) == [4, 3, 3] and sum(fft.compute_budgets([0.2, 0.5, 0.3], 7)) == 7
