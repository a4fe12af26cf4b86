"""Checkpoint-loading behaviours: provenance of the normalisation convention, weights-file resolution with clear
errors, per-group projection remapping by group name, cyclic tiling of widened linear inputs."""

import json

import pytest
import torch
from torch import nn

from helpers import tiny_pi05, tiny_pi05_config
from opentau_b200.policies import loading
from opentau_b200.policies.pi05.modeling_pi05 import PI05Policy


def test_config_version_follows_the_weights(tmp_path):
    pol = tiny_pi05()
    pol.save_pretrained(tmp_path / "ck")
    assert loading.peek_config_version(tmp_path / "ck") == json.loads((tmp_path / "ck/config.json").read_text())["config_version"]
    # a checkpoint that carries only the pipeline config (training checkpoints, published hf_config.json)
    raw = json.loads((tmp_path / "ck/config.json").read_text())
    for name, ver in (("train_config.json", 1), ("hf_config.json", 0)):
        d = tmp_path / name.split(".")[0]
        d.mkdir()
        (d / name).write_text(json.dumps({"policy": {**raw, "config_version": ver}, "steps": 3}))
        assert loading.peek_config_version(d) == ver
    # no tag anywhere: a pre-versioning checkpoint; an explicit value on the config is kept
    legacy = tmp_path / "legacy"
    legacy.mkdir()
    (legacy / "config.json").write_text(json.dumps({k: v for k, v in raw.items() if k != "config_version"}))
    cfg = tiny_pi05_config()
    cfg.config_version = None
    loading.resolve_checkpoint_provenance(cfg, legacy)
    assert cfg.config_version == 0
    cfg.config_version = 1
    loading.resolve_checkpoint_provenance(cfg, legacy)
    assert cfg.config_version == 1
    assert loading.peek_config_version(tmp_path / "does_not_exist") is None


def test_weights_file_resolution_and_errors(tmp_path, monkeypatch):
    pol = tiny_pi05()
    pol.save_pretrained(tmp_path / "ck")
    assert loading.resolve_pretrained_weights_file(tmp_path / "ck").endswith("model.safetensors")
    (tmp_path / "sharded").mkdir()
    with pytest.raises(loading.CheckpointWeightsNotFoundError, match="consolidate"):
        loading.resolve_pretrained_weights_file(tmp_path / "sharded")
    # repo[@revision] against the local cache
    from opentau_b200.utils import hub
    monkeypatch.setattr(hub, "HF_OPENTAU_HOME", tmp_path / "cache")
    repo = tmp_path / "cache" / "org" / "model"
    (repo / "step-000100").mkdir(parents=True)
    (repo / "step-000100" / "model.safetensors").write_bytes(b"x")
    assert loading.resolve_pretrained_weights_file("org/model@100").endswith("step-000100/model.safetensors")
    with pytest.raises(FileNotFoundError, match="step-000100"):
        loading.resolve_pretrained_weights_file("org/model@200")          # lists the cached revisions
    with pytest.raises(FileNotFoundError, match="neither a local path"):
        loading.resolve_pretrained_weights_file("org/other")
    # a directory without weights yields the constructed policy (its weights come with the training state)
    cfgdir = tmp_path / "resume"
    cfgdir.mkdir()
    pol.config._save_pretrained(cfgdir)
    got = PI05Policy.from_pretrained(cfgdir, config=tiny_pi05_config())
    assert isinstance(got, PI05Policy)


def test_per_group_projection_remap_by_name():
    rec = loading.reconcile_projection_tensor
    w = torch.arange(6.0).view(2, 3)
    # a shared layer loaded into 3 groups: duplicated
    out = rec("m.state_proj.weight", w, torch.zeros(3, 2, 3), None, ["a", "b", "c"])
    assert out.shape == (3, 2, 3) and torch.equal(out[2], w)
    # same names, same order: untouched
    g = torch.randn(2, 2, 3)
    assert rec("m.state_proj.weight", g, torch.zeros(2, 2, 3), ["a", "b"], ["a", "b"]) is g
    # re-ordered and extended by name; an unknown group copies row 0
    out = rec("m.state_proj.weight", g, torch.zeros(3, 2, 3), ["a", "b"], ["b", "new", "a"])
    assert torch.equal(out[0], g[1]) and torch.equal(out[1], g[0]) and torch.equal(out[2], g[0])
    # biases carry one axis less
    b = torch.randn(2, 5)
    assert rec("m.state_proj.bias", b, torch.zeros(3, 5), ["a", "b"], ["b", "a", "a"]).shape == (3, 5)
    with pytest.raises(loading.ProjectionRemapError, match="shares one"):
        rec("m.state_proj.weight", g, torch.zeros(2, 3), ["a", "b"], None)
    with pytest.raises(loading.ProjectionRemapError, match="order is unknown"):
        rec("m.state_proj.weight", g, torch.zeros(3, 2, 3), None, ["a", "b", "c"])
    with pytest.raises(loading.ProjectionRemapError, match="does not fit"):
        rec("m.state_proj.weight", torch.zeros(2, 2, 4), torch.zeros(3, 2, 3), ["a", "b"], ["a", "b", "c"])

    class P(nn.Module):
        def __init__(self):
            super().__init__()
            self.state_proj = nn.ParameterDict({"weight": nn.Parameter(torch.zeros(3, 2, 3))})
            self.config = type("C", (), {"dataset_names": ["x", "y", "z"]})()
    pol = P()
    state = {"state_proj.weight": w.clone(), "other.weight": torch.zeros(1)}
    assert loading.remap_per_group_projection_weights(pol, state, ("state_proj.",), None) == ["state_proj.weight"]
    assert state["state_proj.weight"].shape == (3, 2, 3)


def test_linear_inputs_are_tiled_cyclically():
    class P(nn.Module):
        def __init__(self):
            super().__init__()
            self.inp = nn.Linear(7, 4)
            self.same = nn.Linear(3, 4)
    pol = P()
    w = torch.arange(12.0).view(4, 3)
    state = {"inp.weight": w.clone(), "same.weight": torch.zeros(4, 3)}
    assert loading.tile_linear_input_weights(pol, state) == ["inp.weight"]
    assert state["inp.weight"].shape == (4, 7)
    assert torch.equal(state["inp.weight"], torch.cat([w, w, w[:, :1]], 1))
    pol.load_state_dict(state, strict=False)
    with pytest.raises(ValueError, match="output width"):
        loading.tile_linear_input_weights(pol, {"inp.weight": torch.zeros(5, 3)})


def test_repo_revision_specs(tmp_path, monkeypatch):
    import pytest

    from opentau_b200.utils import hub
    assert hub.split_repo_revision("org/run@6000") == ("org/run", "6000")            # the tag as given
    assert hub.split_repo_revision(*hub.split_repo_revision("org/run@6000")) == ("org/run", "6000")   # idempotent
    assert hub.split_repo_revision("org/run") == ("org/run", None)
    assert hub.split_repo_revision("org/run", "main") == ("org/run", "main")
    assert hub.split_repo_revision(None, "x") == (None, "x")
    local = tmp_path / "ck@v2"
    local.mkdir()
    assert hub.split_repo_revision(str(local)) == (str(local), None)                 # existing paths are never split
    moved = "/data/moved/ck@v2/sub"
    assert hub.split_repo_revision(moved) == (moved, None)                           # path-shaped: fails as a path
    with pytest.raises(ValueError, match="conflicting revisions"):
        hub.split_repo_revision("org/run@6000", "7000")
    assert hub.split_repo_revision("org/run@6000", "6000") == ("org/run", "6000")
    with pytest.raises(ValueError, match="malformed"):
        hub.split_repo_revision("org/run@")
    assert hub.format_repo_revision("org/run", "6000") == "org/run@6000" and hub.format_repo_revision("org/run", None) == "org/run"
    # a step may sit in the cache under its tag or under step-<six digits>
    repo = tmp_path / "cache" / "org" / "run"
    (repo / "6000").mkdir(parents=True)
    (repo / "step-000700").mkdir()
    assert hub.cached_revision_dir(repo, "6000").name == "6000"
    assert hub.cached_revision_dir(repo, "700").name == "step-000700"
    assert hub.cached_revision_dir(repo, "9").name == "step-000009" and hub.cached_revision_dir(repo, None) == repo


def test_policies_and_configs_push_one_commit(tmp_path):
    from helpers import tiny_pi05

    class Api:
        def __init__(self):
            self.calls = []

        def create_repo(self, repo_id, private=None, exist_ok=False):
            self.calls.append(("create_repo", repo_id, private, exist_ok))
            return type("R", (), {"repo_id": repo_id})()

        def upload_folder(self, **kw):
            kw["files"] = sorted(p.name for p in kw["folder_path"].iterdir())
            self.calls.append(("upload_folder", kw))
            return f"https://hub/{kw['repo_id']}/commit/abc"
    pol, api = tiny_pi05(), Api()
    url = pol.push_to_hub("org/tiny", private=True, branch="dev", ignore_patterns=["*.tmp"], api=api)
    assert url.endswith("org/tiny/commit/abc") and api.calls[0] == ("create_repo", "org/tiny", True, True)
    up = api.calls[1][1]
    assert up["commit_message"] == "Upload policy" and up["revision"] == "dev" and up["repo_type"] == "model"
    assert "model.safetensors" in up["files"] and "config.json" in up["files"] and up["ignore_patterns"] == ["*.tmp"]
    api2 = Api()
    pol.config.push_to_hub("org/tiny-config", api=api2)
    assert api2.calls[1][1]["commit_message"] == "Upload config" and api2.calls[1][1]["files"] == ["config.json"]
    # save_pretrained alone stays local; with push_to_hub the repository defaults to the folder's name
    assert pol.save_pretrained(tmp_path / "my-run") is None and (tmp_path / "my-run" / "model.safetensors").is_file()
    api3 = Api()
    pol.save_pretrained(tmp_path / "my-run", push_to_hub=True, api=api3)
    assert api3.calls[0][1] == "my-run"
