"""PerGroupLinear, outlier detection, master-weight optimizer."""

import torch

from opentau_b200.optim.master_weights import MasterWeightOptimizer
from opentau_b200.policies.layers import PerGroupLinear, promote_linear_state
from opentau_b200.policies.outlier_utils import detect_state_action_outliers, log_outlier_records


def test_per_group_linear_routes_each_sample_to_its_group():
    torch.manual_seed(0)
    m = PerGroupLinear(6, 4, 3)
    x = torch.randn(5, 7, 6)
    idx = torch.tensor([2, 0, 2, 1, 0])
    y = m(x, idx)
    for b in range(5):
        want = torch.nn.functional.linear(x[b], m.weight[idx[b]], m.bias[idx[b]])
        assert torch.allclose(y[b], want, atol=1e-6)
    y.sum().backward()
    assert m.weight.grad[1].abs().sum() > 0
    one = PerGroupLinear(6, 4, 1)
    assert torch.allclose(one(x), torch.nn.functional.linear(x, one.weight[0], one.bias[0]), atol=1e-6)
    lin = torch.nn.Linear(6, 4)
    sd = promote_linear_state({"p.weight": lin.weight.data, "p.bias": lin.bias.data}, "p", 3)
    assert sd["p.weight"].shape == (3, 4, 6) and torch.equal(sd["p.weight"][2], lin.weight.data)


def test_outlier_detection_respects_padding_and_reports_provenance():
    st = torch.zeros(2, 3, 4)
    st[0, 0, 1] = 99.0            # padded history step: ignored
    st[1, 2, 3] = 50.0            # current frame: reported
    ac = torch.zeros(2, 5, 4)
    ac[0, 4, 0] = -70.0           # padded action step: ignored
    ac[0, 1, 2] = 40.0
    batch = {"state": st, "actions": ac, "obs_history_is_pad": torch.tensor([[True, False, False]] * 2),
             "action_is_pad": torch.tensor([[False] * 4 + [True]] * 2), "dataset_repo_id": ["a", "b"],
             "episode_index": torch.tensor([7, 8]), "frame_index": torch.tensor([70, 80])}
    recs = detect_state_action_outliers(batch, 32.0)
    got = {(r["key"], r["source"], r["dim"]): r for r in recs}
    assert set(got) == {("state", "b", 3), ("actions", "a", 2)}
    assert got[("state", "b", 3)]["value"] == 50.0 and got[("state", "b", 3)]["episode"] == 8
    assert detect_state_action_outliers(batch, None) == [] and detect_state_action_outliers(batch, 100.0) == []
    seen: set = set()
    assert log_outlier_records(recs, 32.0, seen) == 2 and log_outlier_records(recs, 32.0, seen) == 0


def test_master_weights_keep_small_updates_that_bf16_would_lose():
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.ones(64, dtype=torch.bfloat16))
    opt = MasterWeightOptimizer([p], lambda ms: torch.optim.SGD(ms, lr=1e-3))
    for _ in range(20):                       # each step moves by 1e-3: below bf16 resolution at 1.0 (2^-8)
        p.grad = torch.ones_like(p)
        opt.step()
        opt.zero_grad()
    assert abs(float(opt.masters[0][0]) - 0.98) < 1e-5 and float(p[0]) < 1.0
    q = torch.nn.Parameter(torch.ones(64, dtype=torch.bfloat16))
    naive = torch.optim.SGD([q], lr=1e-3)
    for _ in range(20):
        q.grad = torch.ones_like(q)
        naive.step()
    assert float(q[0]) == 1.0                 # the plain bf16 update rounds away
    p.grad = torch.full_like(p, 100.0)
    assert float(opt.clip_grad_norm_(1.0)) > 1.0
    sd = opt.state_dict()
    opt.load_state_dict(sd)


def test_loc_tokens_become_single_tokens_and_grow_other_vocabularies():
    import torch
    from torch import nn
    from opentau_b200.datasets.grounding.tokenizer_utils import LOC_TOKENS, ensure_loc_tokens
    from opentau_b200.utils.tokenizer import HashTokenizer
    pg = HashTokenizer(257152)
    assert len(pg.encode("<loc0007> cup", add_special_tokens=False)) > 2             # fragmented before
    assert ensure_loc_tokens(pg) == 0 and len(pg) == 257152                         # reserved ids, nothing grows
    ids = pg.encode("<loc0007><loc1023> cup", add_special_tokens=False)
    assert ids[:2] == [256007, 257023] and all(i < 256000 for i in ids[2:])
    assert ensure_loc_tokens(pg) == 0

    class Tiny(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed_tokens = nn.Embedding(500, 16)

    small, model = HashTokenizer(500), Tiny()
    old = model.embed_tokens.weight.detach().clone()
    torch.manual_seed(7)
    expect_next = torch.rand(1)
    torch.manual_seed(7)
    assert ensure_loc_tokens(small, model) == 1024 and len(small) == 1524
    assert torch.equal(torch.rand(1), expect_next)                                  # the caller's RNG stream is untouched
    w = model.embed_tokens.weight
    assert w.shape == (1524, 16) and torch.equal(w[:500], old) and w.requires_grad
    again = Tiny()
    ensure_loc_tokens(HashTokenizer(500), again)
    assert torch.equal(again.embed_tokens.weight[500:], w[500:])                    # same new rows on every run
    assert small.encode(LOC_TOKENS[3], add_special_tokens=False) == [503] and ensure_loc_tokens(small, model) == 0


def test_diagnose_host_script_writes_a_report(tmp_path):
    import subprocess
    from pathlib import Path

    import opentau_b200
    script = Path(opentau_b200.__file__).parent / "scripts" / "diagnose_host.sh"
    out = subprocess.run(["bash", str(script), str(tmp_path)], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and "report:" in out.stdout
    reports = list(tmp_path.glob("*_host.txt"))
    assert len(reports) == 1
    text = reports[0].read_text()
    assert "## GPUs" in text and "## python stack" in text and "torch" in text


def test_action_generation_script_sweeps_step_counts(tmp_path):
    import json

    import numpy as np
    from PIL import Image

    from opentau_b200.scripts import run_action_generation as rag
    Image.fromarray(np.random.default_rng(0).integers(0, 255, (96, 160, 3)).astype(np.uint8)).save(tmp_path / "frame.png")
    out = rag.main(["--image", str(tmp_path / "frame.png"), "--prompt", "pick up the cup", "--domain", "droid",
                    "--chunk-size", "10", "--steps", "3,1", "--warmup", "1", "--tiny", "--device", "cpu",
                    "--output", str(tmp_path / "o" / "action.json")])
    saved = json.loads((tmp_path / "o" / "action.json").read_text())
    assert saved["shape"] == [10, 10] and [r["steps"] for r in saved["sweep"]] == [3, 1]
    assert all(r["finite"] and r["latency_s"] > 0 for r in saved["sweep"]) and saved["weights"] == "random initialisation"
    assert np.asarray(out["data"]).shape == (10, 10)
    import pytest
    with pytest.raises(SystemExit, match="unknown --domain"):
        rag.main(["--image", str(tmp_path / "frame.png"), "--domain", "submarine", "--tiny"])


def test_rng_state_round_trip_and_muted_output(capfd):
    import os
    import random

    import numpy as np
    import pytest

    from opentau_b200.utils.io_utils import silence_output_unless_error
    from opentau_b200.utils.random_utils import get_rng_state, set_rng_state
    state = get_rng_state()
    a = (random.random(), float(np.random.rand()), float(torch.rand(1)))
    set_rng_state(state)
    assert (random.random(), float(np.random.rand()), float(torch.rand(1))) == a
    with silence_output_unless_error("quiet"):
        os.write(1, b"banner from a C extension\n")
        os.write(2, b"and its warnings\n")
    out, err = capfd.readouterr()
    assert "banner" not in out + err and "warnings" not in out + err
    # Python-level prints go through file descriptor 1 in a plain process (pytest's capture rewires sys.stdout)
    import subprocess
    import sys
    code = ("from opentau_b200.utils.io_utils import silence_output_unless_error as s\n"
            "with s():\n    print('muted')\nprint('shown')\n")
    run = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=os.getcwd())
    assert run.stdout.strip() == "shown" and run.returncode == 0
    with pytest.raises(RuntimeError, match="boom"):
        with silence_output_unless_error("task=CloseFridge idx=3"):
            os.write(2, b"the reason it failed\n")
            raise RuntimeError("boom")
    out, err = capfd.readouterr()
    assert "task=CloseFridge idx=3" in err and "the reason it failed" in err
    print("still works")
    assert "still works" in capfd.readouterr().out
