"""DCT + BPE action tokenizer: merges compress smooth trajectories, decoding inverts encoding up to quantisation."""

import numpy as np

from opentau_b200.scripts.fit_fast_tokenizer import fit
from opentau_b200.utils.tokenizer import BpeDctActionTokenizer


def _chunks(n=200, T=20, D=4, seed=0):
    rng = np.random.default_rng(seed)
    t = np.linspace(0, 1, T)[None, :, None]
    return rng.uniform(-1, 1, (n, 1, D)) + rng.uniform(-1, 1, (n, 1, D)) * t + 0.3 * np.sin(2 * np.pi * t * rng.integers(1, 3, (n, 1, D)))


def test_fit_compress_and_roundtrip(tmp_path):
    tok, norm, rep = fit(_chunks(), vocab_size=512)
    assert rep["merges"] > 0 and rep["tokens_per_chunk_mean"] < rep["symbols_per_chunk_mean"]
    assert rep["reconstruction_rmse"] < 0.05 and len(norm["q01"]) == 4
    x = np.clip(_chunks(5, seed=7) / 2.5, -1, 1)
    ids = tok(x)
    assert all(0 < i < tok.vocab_size for row in ids for i in row)
    rec = tok.decode(ids)
    assert np.abs(rec - x).max() < 0.15
    tok.save(tmp_path / "t.json")
    again = BpeDctActionTokenizer.load(tmp_path / "t.json")
    assert again(x) == ids and again.vocab_size == tok.vocab_size
