"""Config codec, registries, refs, CLI overrides, pipeline invariants."""

import json

import pytest

from opentau_b200.configs import codec
from opentau_b200.configs.default import DatasetConfig, DatasetMixtureConfig, DistributedConfig
from opentau_b200.configs.parser import filter_distributed_args, parse_config
from opentau_b200.configs.policies import PreTrainedConfig
from opentau_b200.configs.refs import load_json_with_refs
from opentau_b200.configs.train import TrainPipelineConfig
from opentau_b200.configs.types import FeatureType, NormalizationMode
from opentau_b200.optim.optimizers import AdamWConfig, OptimizerConfig
from opentau_b200.optim.schedulers import CosineDecayWithWarmupSchedulerConfig, LRSchedulerConfig


def _base_cfg():
    return {
        "dataset_mixture": {"datasets": [{"synthetic": {"name": "s"}}], "weights": [1.0]},
        "policy": {"type": "pi05", "chunk_size": 10, "n_action_steps": 10, "num_steps": 5,
                   "input_features": {"camera0": {"type": "VISUAL", "shape": [3, 224, 224]},
                                      "state": {"type": "STATE", "shape": [32]}},
                   "output_features": {"actions": {"type": "ACTION", "shape": [32]}}},
        "batch_size": 8, "gradient_accumulation_steps": 2, "steps": 10, "action_chunk": 10,
        "optimizer": {"type": "adamw", "lr": 1e-4, "betas": [0.9, 0.95]},
        "scheduler": {"type": "cosine_decay_with_warmup", "num_warmup_steps": 2, "num_decay_steps": 10,
                      "peak_lr": 1e-4, "decay_lr": 1e-5},
    }


def test_roundtrip_and_registry():
    cfg = TrainPipelineConfig.from_dict(_base_cfg())
    assert cfg.policy.type == "pi05" and cfg.policy.num_steps == 5
    assert isinstance(cfg.optimizer, AdamWConfig) and cfg.optimizer.betas == (0.9, 0.95)
    assert isinstance(cfg.scheduler, CosineDecayWithWarmupSchedulerConfig)
    assert cfg.policy.input_features["camera0"].type is FeatureType.VISUAL
    assert cfg.policy.input_features["camera0"].shape == (3, 224, 224)
    assert cfg.policy.normalization_mapping["STATE"] is NormalizationMode.MIN_MAX
    d = cfg.to_dict()
    assert d["policy"]["type"] == "pi05" and d["optimizer"]["type"] == "adamw"
    cfg2 = TrainPipelineConfig.from_dict(json.loads(json.dumps(d)))
    assert cfg2.to_dict() == d


def test_batch_invariant_and_shape_propagation():
    cfg = TrainPipelineConfig.from_dict(_base_cfg())
    assert cfg.dataloader_batch_size == 4
    assert cfg.policy.chunk_size == 10 and cfg.policy.max_action_dim == 32
    bad = _base_cfg()
    bad["dataloader_batch_size"] = 3
    with pytest.raises(ValueError):
        TrainPipelineConfig.from_dict(bad)
    raw = _base_cfg()
    raw["action_chunk"] = 6
    cfg = TrainPipelineConfig.from_dict(raw)
    assert cfg.policy.chunk_size == 6 and cfg.policy.n_action_steps == 6


def test_unknown_field_and_unknown_type_raise():
    raw = _base_cfg()
    raw["policy"]["not_a_field"] = 1
    with pytest.raises(KeyError):
        TrainPipelineConfig.from_dict(raw)
    raw = _base_cfg()
    raw["policy"]["type"] = "nope"
    with pytest.raises(KeyError):
        TrainPipelineConfig.from_dict(raw)
    assert "adamw" in OptimizerConfig.get_known_choices()
    assert "constant" in LRSchedulerConfig.get_known_choices()


def test_cli_overrides_and_launcher_arg_filter(tmp_path):
    f = tmp_path / "cfg.json"
    f.write_text(json.dumps(_base_cfg()))
    cfg = parse_config(TrainPipelineConfig, [f"--config_path={f}", "--policy.num_steps=3", "--steps=77",
                                              "--local_rank=0", "--dataset_mixture.weights.0=2.5",
                                              "--loss_weighting.CE=0.25"])
    assert cfg.policy.num_steps == 3 and cfg.steps == 77
    assert cfg.dataset_mixture.weights == [2.5]
    assert cfg.loss_weighting["CE"] == 0.25
    assert filter_distributed_args(["--local_rank", "3", "--a=1", "--master_port=99"]) == ["--a=1"]


def test_refs_merge_and_cycle(tmp_path):
    (tmp_path / "frag.json").write_text(json.dumps({"synthetic": {"name": "x"}, "robot_type": "so101"}))
    raw = _base_cfg()
    raw["dataset_mixture"]["datasets"] = [{"$ref": "frag.json", "robot_type": "override"}]
    (tmp_path / "cfg.json").write_text(json.dumps(raw))
    loaded = load_json_with_refs(tmp_path / "cfg.json")
    assert loaded["dataset_mixture"]["datasets"][0] == {"synthetic": {"name": "x"}, "robot_type": "override"}
    (tmp_path / "a.json").write_text(json.dumps({"$ref": "b.json"}))
    (tmp_path / "b.json").write_text(json.dumps({"$ref": "a.json"}))
    with pytest.raises(ValueError):
        load_json_with_refs(tmp_path / "a.json")


def test_dataset_config_validation():
    with pytest.raises(ValueError):
        DatasetConfig()
    with pytest.raises(ValueError):
        DatasetConfig(repo_id="a", vqa="b")
    with pytest.raises(ValueError):
        DatasetConfig(vqa="clevr", prompt_substitutions={"a": ["b"]})
    with pytest.raises(ValueError):
        DatasetConfig(repo_id="a", use_delta_joint_actions=True)
    with pytest.raises(ValueError):
        DatasetMixtureConfig(datasets=[DatasetConfig(repo_id="a")], weights=[1.0, 2.0])


def test_accelerate_yaml_mapping(tmp_path):
    y = tmp_path / "ds.yaml"
    y.write_text("distributed_type: DEEPSPEED\ndeepspeed_config:\n  zero_stage: 3\n  gradient_clipping: 10\n")
    d = DistributedConfig.from_accelerate_yaml(str(y))
    assert d.strategy == "zero3" and d.gradient_clipping == 10.0
    y.write_text("distributed_type: FSDP\n")
    assert DistributedConfig.from_accelerate_yaml(str(y)).strategy == "fsdp"
    y.write_text("distributed_type: MULTI_GPU\n")
    assert DistributedConfig.from_accelerate_yaml(str(y)).strategy == "ddp"


def test_policy_config_save_load_and_version_semantics(tmp_path):
    cfg = TrainPipelineConfig.from_dict(_base_cfg()).policy
    # no version on a fresh config = the current conventions (what a save then stamps, so a reload behaves the same);
    # legacy behaviour needs the explicit 0 that loading pre-version weights resolves to
    assert cfg.config_version is None and cfg.normalization_epsilon == 1e-6 and cfg.zero_range_centers_on_zero
    cfg._save_pretrained(tmp_path)
    saved = json.loads((tmp_path / "config.json").read_text())
    assert saved["config_version"] == 1 and saved["type"] == "pi05"
    loaded = PreTrainedConfig.from_pretrained(tmp_path)
    assert loaded.normalization_epsilon == 1e-6 and loaded.zero_range_centers_on_zero
    assert loaded.num_steps == 5


def test_scheduler_formula():
    s = CosineDecayWithWarmupSchedulerConfig(num_warmup_steps=4, num_decay_steps=20, peak_lr=1.0, decay_lr=0.1)
    f = s.lr_lambda(100)
    assert f(0) == pytest.approx(1 / 5)
    assert f(2) == pytest.approx((1 / 5 - 1) * 0.5 + 1)
    assert f(20) == pytest.approx(0.1) and f(200) == pytest.approx(0.1)
    import math
    assert f(10) == pytest.approx(0.9 * 0.5 * (1 + math.cos(math.pi * 0.5)) + 0.1)


def test_input_resolution_validation(caplog):
    import logging

    import pytest

    from opentau_b200.configs.types import FeatureType, PolicyFeature
    from opentau_b200.policies.factory import make_policy_config

    def cfg(resize, shapes, **kw):
        feats = {f"camera{i}": PolicyFeature(type=FeatureType.VISUAL, shape=(3, *hw)) for i, hw in enumerate(shapes)}
        feats["state"] = PolicyFeature(type=FeatureType.STATE, shape=(8,))
        return make_policy_config("pi05", resize_imgs_with_padding=resize, input_features=feats,
                                  output_features={"actions": PolicyFeature(type=FeatureType.ACTION, shape=(7,))}, **kw)

    cfg((224, 224), [(224, 224), (224, 224)]).validate_input_resolution(strict=True)       # matches: silent
    cfg(None, [(180, 320), (180, 320)]).validate_input_resolution(strict=True)             # native, one geometry
    with pytest.raises(ValueError, match="camera1=\\(180, 320\\)"):
        cfg((224, 224), [(224, 224), (180, 320)]).validate_input_resolution(strict=True)
    with pytest.raises(ValueError, match="mixed resolutions"):
        cfg(None, [(224, 224), (180, 320)]).validate_input_resolution(strict=True)
    with caplog.at_level(logging.WARNING):
        cfg((224, 224), [(180, 320)]).validate_input_resolution(strict=False)              # eval load: warn only
        cfg((224, 224), [(180, 320)], skip_input_resolution_check=True).validate_input_resolution(strict=True)
    assert sum("differs from the bound image features" in r.getMessage() for r in caplog.records) == 2


def test_pipeline_config_location_fallbacks_and_running_best_resolution(tmp_path, monkeypatch):
    """``from_pretrained`` finds ``train_config.json``, falls back to ``hf_config.json``, resolves ``repo@step`` in
    the local cache and names the cached revisions when one is missing; the running-best metric resolves like the
    reference's and is never serialised."""
    import json
    import pytest
    from opentau_b200.configs.train import TrainPipelineConfig
    from opentau_b200.utils import hub
    raw = {"dataset_mixture": {"datasets": [{"synthetic": {"length": 8, "name": "a"}}], "action_freq": 10.0},
           "policy": {"type": "pi05"}, "steps": 7, "batch_size": 2}
    d = tmp_path / "published"
    d.mkdir()
    (d / "hf_config.json").write_text(json.dumps(raw))
    assert TrainPipelineConfig.from_pretrained(d).steps == 7
    (d / "train_config.json").write_text(json.dumps({**raw, "steps": 9}))
    assert TrainPipelineConfig.from_pretrained(d).steps == 9              # the training name wins
    with pytest.raises(FileNotFoundError, match="neither train_config.json nor hf_config.json"):
        (tmp_path / "empty").mkdir()
        TrainPipelineConfig.from_pretrained(tmp_path / "empty")
    monkeypatch.setattr(hub, "HF_OPENTAU_HOME", tmp_path / "cache")
    rev = tmp_path / "cache" / "org" / "run" / "step-000500"
    rev.mkdir(parents=True)
    (rev / "hf_config.json").write_text(json.dumps({**raw, "steps": 500}))
    assert TrainPipelineConfig.from_pretrained("org/run@500").steps == 500
    with pytest.raises(FileNotFoundError, match="step-000500"):
        TrainPipelineConfig.from_pretrained("org/run@123")
    cfg = TrainPipelineConfig.from_dict({**raw, "running_best_count": 1, "val_freq": 5})
    cfg.validate()
    assert cfg.running_best_metric_resolved == "val_loss" and "running_best_metric_resolved" not in cfg.to_dict()
    bad = TrainPipelineConfig.from_dict({**raw, "running_best_count": 1, "running_best_metric": "eval_success"})
    with pytest.raises(ValueError, match="simulation evaluation source"):
        bad.validate()
    with pytest.raises(ValueError, match="must be one of"):
        TrainPipelineConfig.from_dict({**raw, "running_best_metric": "accuracy"}).validate()


def test_policy_config_loads_from_pipeline_files_strips_retired_fields_and_warns(tmp_path):
    """``PreTrainedConfig.from_pretrained``: falls back from config.json to the ``policy`` object of hf_config.json /
    train_config.json, follows ``$ref`` includes, reports deprecated / removed fields and drops them without
    rewriting the source, and a save never writes them back.  A fresh config behaves as the current version."""
    import json
    import warnings

    import pytest

    from helpers import tiny_pi05_config
    from opentau_b200.configs import policies as P
    cfg = tiny_pi05_config()
    assert cfg.config_version is None and cfg.resolved_config_version() == P.CURRENT_CONFIG_VERSION
    assert cfg.zero_range_centers_on_zero and cfg.normalization_epsilon == P.OPENPI_EPS
    cfg.config_version = 0
    assert not cfg.zero_range_centers_on_zero and cfg.normalization_epsilon == P.LEGACY_EPS
    cfg.config_version = None
    cfg._save_pretrained(tmp_path / "a")
    saved = json.loads((tmp_path / "a" / "config.json").read_text())
    assert saved["config_version"] == 1 and not set(saved) & set(P.STRIPPED_FIELDS)
    # the pipeline files: policy nested under "policy", one part of it behind a $ref
    b = tmp_path / "b"
    b.mkdir()
    feats = {"input_features": saved.pop("input_features")}
    (b / "features.json").write_text(json.dumps(feats))
    policy = {**saved, "$ref": "features.json", "init_strategy": "expert_only", "cloud_vlm_latency_mean": 0.2}
    (b / "hf_config.json").write_text(json.dumps({"policy": policy, "steps": 10}))
    before = (b / "hf_config.json").read_text()
    with pytest.warns(DeprecationWarning) as rec:
        loaded = P.PreTrainedConfig.from_pretrained(b)
    text = " | ".join(str(w.message) for w in rec)
    assert "cloud_vlm_latency_mean" in text and "init_strategy" in text
    assert loaded.type == "pi05" and set(loaded.input_features) == set(cfg.input_features)
    assert (b / "hf_config.json").read_text() == before                  # the source is never rewritten
    (b / "config.json").write_text(json.dumps({**saved, **feats, "chunk_size": 7, "n_action_steps": 7}))
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        assert P.PreTrainedConfig.from_pretrained(b).chunk_size == 7     # config.json wins over the pipeline files
    c = tmp_path / "c"
    c.mkdir()
    (c / "train_config.json").write_text(json.dumps({"steps": 10}))
    with pytest.raises(FileNotFoundError, match="no 'policy' object"):
        P.PreTrainedConfig.from_pretrained(c)
    (tmp_path / "d").mkdir()
    with pytest.raises(FileNotFoundError, match="None of config.json, hf_config.json, train_config.json"):
        P.PreTrainedConfig.from_pretrained(tmp_path / "d")
    # files we own are cleaned in place
    (tmp_path / "own.json").write_text(json.dumps({"policy": {"init_strategy": "x", "a": 1}, "action_decoder_latency_std": 1}))
    P.strip_deprecated_fields_from_json(tmp_path / "own.json")
    assert json.loads((tmp_path / "own.json").read_text()) == {"policy": {"a": 1}}


def test_dataset_wandb_and_eval_config_rules():
    """The per-dataset index / delta-action rules (JSON string keys coerced), the W&B resume policy and its init
    keywords, and the evaluation video / seed fields."""
    import pytest

    from opentau_b200.configs.default import DatasetConfig, DatasetMixtureConfig, EvalConfig, WandBConfig
    d = DatasetConfig(repo_id="a/b", use_delta_joint_actions=True, delta_action_state_map={"0": 0, "2": "1"})
    assert d.delta_action_state_map == {0: 0, 2: 1}
    for kw, msg in ((dict(delta_action_state_map={0: 0}), "silently ignored"),
                    (dict(use_delta_joint_actions=True), "requires a non-empty"),
                    (dict(use_delta_joint_actions=True, delta_action_state_map={"x": 0}), "must map int"),
                    (dict(use_delta_joint_actions=True, delta_action_state_map={0: -1}), "non-negative"),
                    (dict(state_index=[0, 1, 1]), r"duplicate indices \[1\]"),
                    (dict(action_index=[]), "non-empty list"),
                    (dict(action_index=[True, 2]), "non-negative ints"),
                    (dict(prompt_substitutions={"t": []}), "non-empty list"),
                    (dict(prompt_substitutions={"t": ["ok", ""]}), "empty or non-string"),
                    (dict(prompt_substitutions={"$ref": ["x"]}), "file include"),
                    (dict(val_split_ratio=1.5), r"\[0, 1\]"), (dict(tolerance_s=-1.0), ">= 0")):
        with pytest.raises(ValueError, match=msg):
            DatasetConfig(repo_id="a/b", **kw)
    with pytest.raises(ValueError, match="only applies to LeRobot"):
        DatasetConfig(vqa="dummy", state_index=[0])
    with pytest.raises(ValueError, match="only applies to LeRobot"):
        DatasetConfig(vqa="dummy", prompt_substitutions={"t": ["u"]})
    for kw, msg in ((dict(n_obs_history=0), "positive integer"), (dict(delta_stats_max_rows=True), "positive integer"),
                    (dict(tolerance_s=-1e-3), ">= 0"), (dict(action_freq=0.0), "positive")):
        with pytest.raises(ValueError, match=msg):
            DatasetMixtureConfig(**kw)
    assert DatasetMixtureConfig().action_freq is None

    w = WandBConfig(run_id="abc", notes="n")
    assert w.to_wandb_kwargs(step=None).get("fork_from") is None
    kw = w.to_wandb_kwargs(step=40)
    assert kw["fork_from"] == "abc?_step=40" and kw["notes"].endswith("Forked from run abc at step 40.") and "id" not in kw
    kw = WandBConfig(run_id="abc", on_resume="continue").to_wandb_kwargs(step=40)
    assert kw["id"] == "abc" and kw["resume"] == "allow" and "fork_from" not in kw
    kw = WandBConfig(run_id="abc", mode="offline").to_wandb_kwargs(step=40)
    assert "fork_from" not in kw and "would fork from run abc" in kw["notes"]
    with pytest.warns(FutureWarning, match="deprecated"):
        assert WandBConfig(allow_resume=True).on_resume == "continue"
    with pytest.raises(ValueError, match="on_resume"):
        WandBConfig(on_resume="restart")

    e = EvalConfig(seed_list="3, 5,8", n_episodes=16, batch_size=16)
    assert e.seed_list == [3, 5, 8] and e.n_episodes == 3 and e.batch_size == 3 and e.decorrelate_rank_seeds is False
    for kw, msg in ((dict(video_crf=60), "video_crf"), (dict(video_frame_stride=0), "video_frame_stride"),
                    (dict(video_preset="warp"), "video_preset"), (dict(batch_size=8, n_episodes=4), "batch size")):
        with pytest.raises(ValueError, match=msg):
            EvalConfig(**kw)


def test_cli_help_and_plain_dataclass_configs(tmp_path, capsys):
    """``--help`` lists the dotted fields and exits 0; a config class without ``from_dict`` / ``from_pretrained`` (the
    tools' own small dataclasses) is built by the generic decoder, from overrides alone or from a JSON file."""
    import json
    from dataclasses import dataclass, field

    import pytest

    from opentau_b200.configs import parser
    from opentau_b200.configs.train import TrainPipelineConfig

    @dataclass
    class Inner:
        rate: float = 0.5

    @dataclass
    class ToolConfig:
        root: str = ""
        count: int = 3
        inner: Inner = field(default_factory=Inner)

    with pytest.raises(SystemExit) as e:
        parser.parse_config(ToolConfig, ["--help"], doc="A tool.")
    out = capsys.readouterr().out
    assert e.value.code == 0 and "A tool." in out and "--count=<int>  (default 3)" in out and "--inner.rate=<float>" in out
    with pytest.raises(SystemExit):
        parser.parse_config(TrainPipelineConfig, ["-h"])
    out = capsys.readouterr().out
    assert "--dataset_mixture.*" in out and "--batch_size=" in out and "--eval.n_episodes=" in out
    cfg = parser.parse_config(ToolConfig, ["--root=/data", "--inner.rate=0.25", "--local_rank=1"])
    assert (cfg.root, cfg.count, cfg.inner.rate) == ("/data", 3, 0.25)
    (tmp_path / "tool.json").write_text(json.dumps({"count": 7, "inner": {"rate": 0.1}}))
    cfg = parser.parse_config(ToolConfig, [f"--config_path={tmp_path / 'tool.json'}", "--count=9"])
    assert (cfg.count, cfg.inner.rate) == (9, 0.1)


def test_policy_path_without_a_config_file_and_features_from_the_checkpoint(tmp_path):
    """``--policy.path=<checkpoint>`` alone builds the policy block from the checkpoint's own configuration; a pipeline
    config that only names ``policy.pretrained_path`` (an eval started from the training config, whose policy block
    binds no features) gets its features from the checkpoint too."""
    from helpers import TINY, tiny_pi05
    from opentau_b200.configs import parser
    from opentau_b200.configs.train import TrainPipelineConfig
    from opentau_b200.policies.factory import make_policy
    tiny_pi05().save_pretrained(tmp_path / "ck")
    cfg = parser.parse_config(TrainPipelineConfig, [f"--policy.path={tmp_path / 'ck'}", "--policy.num_steps=3",
                                                    "--resolution=[224,224]", "--num_cams=1"])
    assert cfg.policy.type == "pi05" and cfg.policy.num_steps == 3 and cfg.policy.pretrained_path == str(tmp_path / "ck")
    assert "actions" in cfg.policy.output_features and "state" in cfg.policy.input_features
    bare = TrainPipelineConfig.from_dict({"policy": {"type": "pi05", "pretrained_path": str(tmp_path / "ck"),
                                                     "chunk_size": 10, "n_action_steps": 10, "prompt_max_length": 16,
                                                     "discrete_action_max_length": 8, "discrete_action_vocab_size": 256,
                                                     "device": "cpu", **TINY},
                                          "resolution": [224, 224], "num_cams": 1})
    assert not bare.policy.output_features
    pol = make_policy(bare.policy)
    assert "actions" in pol.unnormalize_outputs.features and "state" in pol.normalize_inputs.features


def test_training_config_checks_data_against_policy(caplog):
    import logging

    import pytest

    from helpers import TINY
    from opentau_b200.configs.train import TrainPipelineConfig

    def build(**kw):
        pol = {"type": "pi05", "chunk_size": 10, "n_action_steps": 10, "prompt_max_length": 16, "device": "cpu",
               "discrete_action_max_length": 8, "discrete_action_vocab_size": 256, **TINY, **kw.pop("policy", {})}
        raw = {"dataset_mixture": {"datasets": [{"synthetic": {"length": 8}}], "action_freq": 10.0, **kw.pop("mix", {})},
               "policy": pol, "resolution": [224, 224], "num_cams": 1, "action_chunk": 10, "batch_size": 2,
               "output_dir": "/tmp/never-created-by-this-test", **kw}
        return TrainPipelineConfig.from_dict(raw)
    build().validate()
    with pytest.raises(ValueError, match="a second time"):
        build(policy={"resize_imgs_with_padding": [448, 448]}).validate()
    with caplog.at_level(logging.WARNING):
        build(policy={"resize_imgs_with_padding": [448, 448], "skip_input_resolution_check": True}).validate()
    assert "Proceeding because skip_input_resolution_check=true" in caplog.text
    with pytest.raises(ValueError, match="missing \\['CE'\\]"):
        build(loss_weighting={"MSE": 1.0}).validate()
    with pytest.raises(ValueError, match="negative entries"):
        build(loss_weighting={"MSE": 1.0, "CE": -0.1}).validate()
    with pytest.raises(ValueError, match="all-zero"):
        build(loss_weighting={"MSE": 0.0, "CE": 0.0}).validate()
    build(loss_weighting={"MSE": 1.0, "CE": 0.0}).validate()                   # one term dropped on purpose
    caplog.clear()
    with caplog.at_level(logging.WARNING):
        cfg = build(policy={"chunk_size": 20, "n_action_steps": 10})
    assert cfg.policy.chunk_size == 10 and "overriding policy.chunk_size=20 with action_chunk=10" in caplog.text
