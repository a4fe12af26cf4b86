"""Normalisation heads keyed by (robot_type, control_mode), their resolution from a batch, delta joint actions from the
dataset columns to the policy's inverse, and the statistics that go with them."""

import json
import logging

import numpy as np
import pytest
import torch

from helpers import tiny_batch, tiny_pi05, tiny_pi05_config
from opentau_b200.datasets.action_indexing import (add_chunk_start_state, apply_column_index, resolve_delta_map,
                                                   subtract_chunk_start_state)
from opentau_b200.datasets.compute_stats import aggregate_feature_stats, aggregate_stats
from opentau_b200.datasets.dataset_mixture import DatasetMixtureMetadata, compute_norm_key
from opentau_b200.datasets.delta_action_stats import (compute_delta_stats_from_columns, delta_stats_cache_key,
                                                      gather_chunks, load_or_compute_delta_stats, select_anchor_rows)
from opentau_b200.datasets.synthetic import identity_stats
from opentau_b200.policies.factory import load_norm_stats_override, make_policy


def test_norm_key_rules():
    assert compute_norm_key("franka", "joint", "repo/a") == ("franka::joint", False)
    assert compute_norm_key(" Franka ", "EE", "repo/a") == ("Franka::EE", False)          # casing kept, blanks trimmed
    for rt, cm in ((None, "joint"), ("franka", ""), ("UNKNOWN", "joint"), ("franka", "Unknown"), ("  ", "joint")):
        assert compute_norm_key(rt, cm, "repo/a") == ("repo/a", True)


class _Member:
    """The attributes the mixture metadata reads from a dataset."""

    def __init__(self, robot_type, control_mode, mean, frames, width=4, delta=None, is_vqa=False, total=8):
        self.robot_type, self.control_mode = robot_type, control_mode
        v = lambda x: np.full(total, x, np.float32) * (np.arange(total) < width)           # noqa: E731
        self.stats = {k: {"mean": v(mean), "std": v(1.0), "min": v(mean - 2), "max": v(mean + 2),
                          "count": np.array([frames])} for k in ("state", "actions")}
        from opentau_b200.configs.types import FeatureType, PolicyFeature
        self.policy_features = {"state": PolicyFeature(FeatureType.STATE, (8,)), "actions": PolicyFeature(FeatureType.ACTION, (8,))}
        self.delta_action_state_map = delta
        self.is_vqa = is_vqa
        self._frames = frames
        self.state_index = self.action_index = list(range(width))

    def __len__(self):
        return self._frames


def test_heads_are_shared_by_robot_and_control_mode_and_pooled_by_frames(caplog):
    a, b = _Member("franka", "joint", 0.0, 100), _Member("franka", "joint", 3.0, 300)
    c, d = _Member("franka", "ee", 5.0, 50), _Member(None, "joint", 7.0, 10)
    with caplog.at_level(logging.INFO):
        meta = DatasetMixtureMetadata([a, b, c, d], ["A", "B", "C", "D"])
    assert meta.norm_keys == ["franka::joint", "franka::ee", "D"]
    assert meta.dataset_to_norm_index == {"A": 0, "B": 0, "C": 1, "D": 2}
    assert meta.norm_key_to_dataset_names["franka::joint"] == ["A", "B"]
    pooled = meta.per_norm_key_stats[0]["actions"]
    assert np.allclose(pooled["mean"][:4], 0.25 * 0.0 + 0.75 * 3.0)                       # frame-weighted
    assert np.allclose(pooled["min"][:4], -2.0) and np.allclose(pooled["max"][:4], 5.0)
    assert meta.per_norm_key_stats[1] is c.stats                                          # a singleton is passed through
    assert "no usable (robot_type, control_mode)" in caplog.text and "'D'" in caplog.text
    assert "normalisation heads: 3 over 4" in caplog.text
    # members of one real pair must agree on the raw widths
    with pytest.raises(ValueError, match="different raw"):
        DatasetMixtureMetadata([a, _Member("franka", "joint", 0.0, 10, width=6)], ["A", "E"])


def test_mixture_delta_map_must_be_one_convention():
    on = _Member("r", "joint", 0.0, 10, delta={0: 0, 1: 1})
    assert DatasetMixtureMetadata([on, _Member("r", "joint", 0.0, 10, delta={1: 1, 0: 0})], ["a", "b"]) \
        .delta_action_state_map == {0: 0, 1: 1}
    assert DatasetMixtureMetadata([on, _Member("q", "x", 0.0, 10, is_vqa=True)], ["a", "v"]).delta_action_state_map
    with pytest.raises(ValueError, match="do not"):
        DatasetMixtureMetadata([on, _Member("r", "joint", 0.0, 10)], ["a", "b"])
    with pytest.raises(ValueError, match="disagree"):
        DatasetMixtureMetadata([on, _Member("r", "joint", 0.0, 10, delta={0: 1})], ["a", "b"])
    assert DatasetMixtureMetadata([_Member("r", "joint", 0.0, 10)], ["a"]).delta_action_state_map is None


def test_aggregation_tolerates_non_finite_dims_and_drops_partial_quantiles(caplog):
    one = {"mean": np.array([1.0, np.nan]), "std": np.array([1.0, 1.0]), "min": np.array([0.0, -np.inf]),
           "max": np.array([2.0, 3.0]), "count": np.array([10]), "q01": np.array([0.1, 0.1]), "q99": np.array([1.9, 1.9])}
    two = {"mean": np.array([3.0, 5.0]), "std": np.array([1.0, 2.0]), "min": np.array([1.0, 4.0]),
           "max": np.array([5.0, 6.0]), "count": np.array([30])}
    with caplog.at_level(logging.WARNING):
        out = aggregate_feature_stats([one, two], contributor_names=["one", "two"], context="head 'x'")
    assert np.allclose(out["mean"], [2.5, 5.0]) and np.allclose(out["min"], [0.0, 4.0]) and out["count"][0] == 40
    assert np.allclose(out["std"][1], 2.0)                     # the NaN contributor is left out of dim 1 only
    assert "q01" not in out and "q99" not in out
    assert "head 'x'" in caplog.text and "'two'" in caplog.text
    both = aggregate_feature_stats([one, {**two, "q01": np.array([0.5, 0.5]), "q99": np.array([4.0, 4.0])}])
    assert np.allclose(both["q01"], [0.4, 0.4])
    with pytest.raises(ValueError, match="parallel"):
        aggregate_feature_stats([one], weights=[1.0, 2.0])
    agg = aggregate_stats([{"a": one}, {"a": two, "b": two}], weights=[1.0, 1.0])
    assert np.allclose(agg["a"]["mean"][0], 2.0) and np.allclose(agg["b"]["mean"], two["mean"])


def test_delta_map_translation_between_index_spaces(caplog):
    # stored layout: actions [x, y, z, grip], state [grip, z, y, x]; emitted: actions [z, x, grip], state [x, z]
    assert resolve_delta_map({0: 3, 2: 1}, action_index=[2, 0, 3], state_index=[3, 1], who="t") == {1: 0, 0: 1}
    assert resolve_delta_map({"0": "1"}, None, None) == {0: 1}
    with pytest.raises(ValueError, match="does not keep"):
        resolve_delta_map({1: 0}, action_index=[0, 2], state_index=None, who="t")
    with pytest.raises(ValueError, match="drops"):
        resolve_delta_map({0: 2}, action_index=None, state_index=[0, 1], who="t")
    with caplog.at_level(logging.WARNING):
        resolve_delta_map({0: 0}, None, None, who="t", action_dim=3)
    assert "[1, 2]" in caplog.text and "ABSOLUTE" in caplog.text
    with pytest.raises(IndexError, match=r"column\(s\) \[7\]"):
        apply_column_index(torch.zeros(2, 4), [0, 7], what="state", who="t")


def test_chunk_start_offsets_all_shapes():
    a, st = torch.randn(2, 5, 4), torch.randn(2, 3)
    d = subtract_chunk_start_state(a, st, {1: 2, 3: 0})
    assert torch.allclose(d[..., 1], a[..., 1] - st[:, 2:3]) and torch.allclose(d[..., 3], a[..., 3] - st[:, 0:1])
    assert torch.equal(d[..., 0], a[..., 0]) and torch.allclose(add_chunk_start_state(d, st, {1: 2, 3: 0}), a, atol=1e-6)
    hist = torch.randn(2, 4, 3)                                    # a history axis: the last step anchors the chunk
    assert torch.allclose(subtract_chunk_start_state(a, hist, {0: 1}), subtract_chunk_start_state(a, hist[:, -1], {0: 1}))
    assert torch.allclose(subtract_chunk_start_state(a[0], hist[0], {0: 1}), subtract_chunk_start_state(a, hist, {0: 1})[0])
    assert subtract_chunk_start_state(a, st, None) is a
    with pytest.raises(IndexError):
        subtract_chunk_start_state(a, st, {5: 0})


def _columns(seed=0, episodes=(30, 45, 25), sd=3, ad=4):
    rng = np.random.default_rng(seed)
    n = sum(episodes)
    ep = np.concatenate([np.full(k, i) for i, k in enumerate(episodes)])
    state = np.cumsum(rng.normal(size=(n, sd)) * 0.1, axis=0)
    action = np.concatenate([state + rng.normal(size=(n, sd)) * 0.05, rng.uniform(0, 1, (n, 1))], axis=1)[:, :ad]
    return state, action, ep


def test_delta_statistics_from_columns_match_a_direct_evaluation():
    state, action, ep = _columns()
    offsets, dm = np.arange(6, dtype=np.float64), {0: 0, 1: 1, 2: 2}
    got = compute_delta_stats_from_columns(state, action, ep, delta_map=dm, chunk_offsets=offsets, block_frames=17)
    rows = []
    for e in np.unique(ep):
        idx = np.flatnonzero(ep == e)
        for t in idx:
            chunk = action[np.clip(t + np.arange(6), idx[0], idx[-1])].copy()       # past the end: the last row repeats
            chunk[:, :3] -= state[t]
            rows.append(chunk)
    flat = np.concatenate(rows)
    assert int(got["actions"]["count"][0]) == len(flat)
    for k, ref in (("mean", flat.mean(0)), ("std", flat.std(0)), ("min", flat.min(0)), ("max", flat.max(0))):
        assert np.allclose(got["actions"][k], ref, atol=1e-5), k
    width = (flat.max(0) - flat.min(0)) / 5000               # one histogram bucket
    for name, q in (("q01", 0.01), ("q99", 0.99)):
        below = (flat <= got["actions"][name] + width).mean(0)
        under = (flat < got["actions"][name] - width).mean(0)
        assert np.all(below >= q - 1e-9) and np.all(under <= q + 1e-9), name
    assert np.allclose(got["state"]["mean"], state.mean(0), atol=1e-6)
    # the deltas are much narrower than the absolute actions on the mapped dims, the gripper dim is untouched
    assert np.all(got["actions"]["std"][:3] < action.std(0)[:3]) and np.isclose(got["actions"]["max"][3], action[:, 3].max())
    # column selection happens before the map is applied (post-index positions)
    sel = compute_delta_stats_from_columns(state, action, ep, delta_map={0: 1}, chunk_offsets=offsets,
                                           state_index=[2, 0], action_index=[0, 3], episodes={1})
    assert sel["actions"]["mean"].shape == (2,) and int(sel["state"]["count"][0]) == 45


def test_anchor_cap_is_a_stride_over_all_episodes_and_linear_resampling_interpolates():
    spans = [(0, 30), (30, 75), (75, 100)]
    full = select_anchor_rows(spans, None)
    assert sum(len(r) for r, _, _ in full) == 100
    capped = select_anchor_rows(spans, 12)
    rows = np.concatenate([r for r, _, _ in capped])
    assert len(rows) <= 12 and len(capped) == 3 and np.all(np.diff(rows) == np.diff(rows)[0])     # one phase throughout
    assert [(lo, hi) for _, lo, hi in capped] == spans                                            # true bounds travel
    vals = np.arange(10, dtype=np.float64)[:, None] * 2.0
    got = gather_chunks(vals, np.array([7.0]), np.array([0.0, 0.5, 1.5, 4.0]), 0, 10, "linear")[0, :, 0]
    assert np.allclose(got, [14.0, 15.0, 17.0, 18.0])
    assert np.allclose(gather_chunks(vals, np.array([7.0]), np.array([0.4, 0.6]), 0, 10, "nearest")[0, :, 0], [14.0, 16.0])
    with pytest.raises(ValueError):
        gather_chunks(vals, np.array([0.0]), np.array([0.0]), 0, 10, "cubic")


def test_delta_statistics_cache(tmp_path):
    kw = dict(state_index=None, action_index=[0, 1], delta_map={0: 0}, chunk_offsets=[0.0, 1.0], episodes=[0, 1],
              vector_resample_strategy="nearest", excluded_episodes=None, fps=30, revision=None)
    key = delta_stats_cache_key(**kw)
    assert key == delta_stats_cache_key(**{**kw, "delta_map": {"0": "0"}, "chunk_offsets": [0.0, 1.0000000001]})
    assert key != delta_stats_cache_key(**{**kw, "chunk_offsets": [0.0, 2.0]})
    assert key != delta_stats_cache_key(**kw, max_rows=100) and len(key) == 12
    calls = []

    def compute():
        calls.append(1)
        state, action, ep = _columns()
        return compute_delta_stats_from_columns(state, action, ep, delta_map={0: 0}, chunk_offsets=[0.0, 1.0])

    first = load_or_compute_delta_stats(tmp_path, key, compute)
    again = load_or_compute_delta_stats(tmp_path, key, compute)
    assert len(calls) == 1 and np.allclose(first["actions"]["q99"], again["actions"]["q99"])
    assert again["actions"]["count"].dtype == np.int64
    f = tmp_path / "meta" / "delta_action_stats" / f"{key}.json"
    f.write_text("{ torn")                                             # an unreadable file is a cache miss
    load_or_compute_delta_stats(tmp_path, key, compute)
    assert len(calls) == 2 and json.loads(f.read_text())["version"] == 1


def _two_head_policy(**over):
    cfg = tiny_pi05_config(**over)
    s1, s2 = identity_stats(), identity_stats()
    for k in s2:
        s2[k] = {n: (v * 2.0 if n in ("std", "max", "min") else v) for n, v in s2[k].items()}
    return make_policy(cfg, per_dataset_stats=[s1, s2], dataset_names=["franka::joint", "so101::ee"]), cfg


def test_dataset_index_resolution_routes():
    pol, cfg = _two_head_policy()
    cfg.dataset_to_norm_index = {"repo/a": 0, "repo/b": 0, "repo/c": 1}
    b = {k: v for k, v in tiny_batch().items() if k != "dataset_index"}
    B = b["state"].shape[0]
    assert pol._stacked_num_datasets() == 2
    assert pol._resolve_dataset_index({**b, "dataset_index": [1] * B}).tolist() == [1] * B
    assert pol._resolve_dataset_index({**b, "robot_type": "so101", "control_mode": "ee"}).tolist() == [1] * B
    mixed = pol._resolve_dataset_index({**b, "robot_type": ["franka"] + ["so101"] * (B - 1), "control_mode": ["joint"] + ["ee"] * (B - 1)})
    assert mixed.tolist() == [0] + [1] * (B - 1)
    assert pol._resolve_dataset_index({**b, "dataset_repo_id": "repo/b"}).tolist() == [0] * B
    # both given: the pair wins over the repository name
    assert pol._resolve_dataset_index({**b, "robot_type": "so101", "control_mode": "ee", "dataset_repo_id": "repo/a"}).tolist() == [1] * B
    with pytest.raises(ValueError, match="not one of"):
        pol._resolve_dataset_index({**b, "robot_type": "so101", "control_mode": "unknown"})
    with pytest.raises(ValueError, match="training set"):
        pol._resolve_dataset_index({**b, "dataset_repo_id": "repo/zzz"})
    with pytest.raises(KeyError, match="2 heads"):
        pol._resolve_dataset_index(b)
    cfg.dataset_names = cfg.dataset_to_norm_index = None               # a multi-head policy that lost its tables
    with pytest.raises(RuntimeError, match="no `dataset_names`"):
        pol._resolve_dataset_index({**b, "dataset_repo_id": "repo/a"})
    single = tiny_pi05()
    single.config.dataset_names = single.config.dataset_to_norm_index = None
    assert single._resolve_dataset_index({**b, "robot_type": "x", "control_mode": "y"}).tolist() == [0] * B
    assert single._resolve_dataset_index(b).tolist() == [0] * B


def test_policy_inverts_delta_actions_and_takes_raw_prefixes():
    pol = tiny_pi05().eval()
    cfg = pol.config
    b = {k: v for k, v in tiny_batch().items() if k != "dataset_index"}
    B = b["state"].shape[0]
    torch.manual_seed(0)
    noise = torch.randn(B, cfg.chunk_size, cfg.max_action_dim)
    absolute = pol.sample_actions(b, noise=noise)
    cfg.delta_action_state_map = {0: 1, 2: 0}
    shifted = pol.sample_actions(b, noise=noise)
    st = b["state"].float()
    st = st[:, -1] if st.dim() == 3 else st
    d = shifted - absolute
    assert torch.allclose(d[..., 0], st[:, 1:2].expand(-1, d.shape[1]), atol=1e-5)
    assert torch.allclose(d[..., 2], st[:, 0:1].expand(-1, d.shape[1]), atol=1e-5) and float(d[..., 1].abs().max()) == 0.0
    # the frozen rows come back as they went in: absolute -> delta -> normalised -> model -> un-normalised -> absolute
    prefix = torch.zeros(B, cfg.chunk_size, cfg.max_action_dim)
    prefix[:, :3, :shifted.shape[-1]] = shifted[:, :3]
    again = pol.sample_actions(b, noise=noise, action_prefix=prefix, delay=3)
    assert torch.allclose(again[:, :3], shifted[:, :3], atol=1e-4)
    with pytest.raises(KeyError, match="no 'state'"):
        pol.sample_actions({k: v for k, v in b.items() if k != "state"}, noise=noise)
    with pytest.raises(ValueError, match="non-negative"):
        tiny_pi05_config(delta_action_state_map={0: -1})
    assert tiny_pi05_config(delta_action_state_map={"3": "1"}).delta_action_state_map == {3: 1}


def test_make_policy_statistics_sources(tmp_path):
    meta = DatasetMixtureMetadata([_Member("franka", "joint", 0.0, 10, width=8, delta={0: 0}, total=32),
                                   _Member("franka", "joint", 1.0, 30, width=8, delta={0: 0}, total=32)], ["A", "B"])
    cfg = tiny_pi05_config()
    pol = make_policy(cfg, ds_meta=meta)
    assert cfg.dataset_names == ["franka::joint"] and cfg.dataset_to_norm_index == {"A": 0, "B": 0}
    assert cfg.delta_action_state_map == {0: 0} and cfg.config_version is not None
    assert not pol._norm_buffers_have_inf()
    # a policy type without the field refuses a delta-action mixture
    from opentau_b200.policies.factory import make_policy_config
    import test_value_cpu
    with pytest.raises(ValueError, match="delta joint actions"):
        make_policy(test_value_cpu._cfg(), ds_meta=meta)
    # caller-supplied opaque statistics: heads are named, no dataset table
    cfg2 = tiny_pi05_config()
    make_policy(cfg2, stats=[identity_stats(), identity_stats()])
    assert cfg2.dataset_names == ["external_0", "external_1"] and cfg2.dataset_to_norm_index is None
    # one file for every head
    f = tmp_path / "norm_stats.json"
    ones = [1.0] * 8
    f.write_text(json.dumps({"norm_stats": {"state": {"mean": ones, "std": ones, "min": ones, "max": ones},
                                            "actions": {"mean": ones, "std": ones, "min": ones, "max": ones}}}))
    heads = load_norm_stats_override(str(f), num_heads=3)
    assert len(heads) == 3 and heads[0]["state"] is not heads[1]["state"]
    f.write_text(json.dumps({"norm_stats": {"state": {}}}))
    with pytest.raises(KeyError, match="actions"):
        load_norm_stats_override(str(f), 1)
    with pytest.raises(ValueError, match="execution_target"):
        make_policy(tiny_pi05_config(), per_dataset_stats=[identity_stats()], execution_target="edge")


def test_missing_statistics_are_reported_at_construction(tmp_path):
    pol = tiny_pi05()
    pol.config.save_normalization_stats = False
    pol.save_pretrained(tmp_path / "ck")
    cfg = tiny_pi05_config(pretrained_path=str(tmp_path / "ck"))
    with pytest.raises(RuntimeError, match=r"still \+inf"):
        make_policy(cfg)
    cfg = tiny_pi05_config(pretrained_path=str(tmp_path / "ck"))
    filled = make_policy(cfg, per_dataset_stats=[identity_stats()])
    assert not filled._norm_buffers_have_inf()


def test_tokenizer_convention_sidecar(tmp_path):
    pol = tiny_pi05()
    tok = tmp_path / "tok"
    tok.mkdir()
    pol._check_discrete_action_tokenizer_convention(tok)                    # no sidecar: no claim
    current = bool(pol.config.zero_range_centers_on_zero)
    (tok / "opentau_action_norm.json").write_text(json.dumps({"config_version": 1, "zero_range_center": current}))
    pol._check_discrete_action_tokenizer_convention(tok)
    (tok / "opentau_action_norm.json").write_text(json.dumps({"config_version": 0, "zero_range_center": not current}))
    with pytest.raises(ValueError, match="mismatch"):
        pol._check_discrete_action_tokenizer_convention(tok)
    (tok / "opentau_action_norm.json").write_text("not json")
    pol._check_discrete_action_tokenizer_convention(tok)                    # unreadable: no claim


def test_inference_batches_are_tagged_from_the_config_section():
    from opentau_b200.configs.default import EvalConfig
    from opentau_b200.configs.deployment import ServerConfig, tag_norm_head
    assert tag_norm_head({}, ServerConfig()) == {}
    assert tag_norm_head({}, ServerConfig(dataset_repo_id="repo/a")) == {"dataset_repo_id": "repo/a"}
    both = tag_norm_head({}, EvalConfig(robot_type="so101", control_mode="ee", dataset_repo_id="repo/a"))
    assert both == {"robot_type": "so101", "control_mode": "ee"}                    # the pair wins
    assert tag_norm_head({}, ServerConfig(robot_type="so101")) == {}                # half a pair names nothing
    assert tag_norm_head({"x": 1}, None) == {"x": 1}
    with pytest.raises(ValueError, match="max_send_message_length_mb"):
        ServerConfig(max_send_message_length_mb=0)


def test_stored_statistics_can_be_dropped_or_promoted_on_load(tmp_path, caplog):
    from safetensors.torch import load_file, save_file
    from opentau_b200.policies.pretrained import is_norm_buffer_key
    assert is_norm_buffer_key("normalize_inputs.buffer_state.mean") and is_norm_buffer_key("module.unnormalize_outputs.buffer_actions.std")
    assert not is_norm_buffer_key("model.normalizer.weight")
    pol = tiny_pi05()
    pol.save_pretrained(tmp_path / "ck")
    # fine-tuning on other data: the checkpoint's statistics are ignored, the fresh ones survive, the flag is consumed
    fresh = identity_stats()
    fresh["state"] = {k: (v + 3.0 if k != "count" else v) for k, v in fresh["state"].items()}
    cfg = tiny_pi05_config(pretrained_path=str(tmp_path / "ck"), skip_normalization_weights=True)
    with caplog.at_level(logging.INFO):
        loaded = make_policy(cfg, per_dataset_stats=[fresh])
    assert "dropped" in caplog.text and cfg.skip_normalization_weights is False
    name = next(iter(loaded.normalize_inputs.buffer_state.keys()))
    assert float(loaded.normalize_inputs.buffer_state[name][0, 0]) == float(fresh["state"][name][0])
    assert float(pol.normalize_inputs.buffer_state[name][0, 0]) == float(fresh["state"][name][0]) - 3.0
    with pytest.raises(ValueError, match="needs `per_dataset_stats`"):
        make_policy(tiny_pi05_config(pretrained_path=str(tmp_path / "ck"), skip_normalization_weights=True))
    # a checkpoint from before the stacked layout: (*feature_shape,) becomes the one row
    f = tmp_path / "ck" / "model.safetensors"
    state = load_file(str(f))
    legacy = {k: (v[0].contiguous() if is_norm_buffer_key(k) else v) for k, v in state.items()}
    save_file(legacy, str(f))
    caplog.clear()
    with caplog.at_level(logging.WARNING):
        old = make_policy(tiny_pi05_config(pretrained_path=str(tmp_path / "ck")))
    assert "promoted" in caplog.text and not old._norm_buffers_have_inf()


def test_zero_variance_guard_reports_real_deviations_once(caplog):
    from opentau_b200.configs.types import FeatureType, NormalizationMode, PolicyFeature
    from opentau_b200.policies import normalize as nz
    nz._WARNED_SNAPS.clear()
    stats = {"state": {"mean": np.array([1.0, 5.0, 0.0], np.float32), "std": np.array([2.0, 0.0, 0.0], np.float32),
                       "min": np.array([0.0, 5.0, 0.0], np.float32), "max": np.array([2.0, 5.0, 0.0], np.float32)}}
    feats = {"state": PolicyFeature(FeatureType.STATE, (3,))}
    for mode in (NormalizationMode.MEAN_STD, NormalizationMode.MIN_MAX):
        nz._WARNED_SNAPS.clear()
        caplog.clear()
        norm = nz.Normalize(feats, {"STATE": mode}, per_dataset_stats=[stats], dataset_names=["arm::joint"])
        with caplog.at_level(logging.WARNING):
            ok = norm({"state": torch.tensor([[1.0, 5.0, 0.0]])})["state"]            # constant dims hold their constant
            assert "zero-variance" not in caplog.text and torch.isfinite(ok).all()
            bad = norm({"state": torch.tensor([[1.0, 5.5, 0.0]])})["state"]           # dim 1 deviates by 0.5
        assert "dim(s) [1]" in caplog.text and "arm::joint" in caplog.text
        assert float(bad.abs().max()) < 10.0                                           # no division by ~eps
        caplog.clear()
        with caplog.at_level(logging.WARNING):
            norm({"state": torch.tensor([[1.0, 5.3, 0.0]])})                          # smaller than already reported
            assert "zero-variance" not in caplog.text
            norm({"state": torch.tensor([[1.0, 7.0, 0.0]])})                          # larger: reported again
            assert "zero-variance" in caplog.text
    healthy = nz.Normalize(feats, {"STATE": NormalizationMode.MEAN_STD}, per_dataset_stats=[
        {"state": {k: np.ones(3, np.float32) for k in ("mean", "std", "min", "max")}}])
    healthy({"state": torch.zeros(1, 3)})
    assert healthy._snap_active is False
    # QUANTILE never degrades to min / max
    with pytest.raises(KeyError, match="QUANTILE normalisation needs"):
        nz.Normalize(feats, {"STATE": NormalizationMode.QUANTILE}, per_dataset_stats=[stats])
    caplog.clear()
    nz._WARNED_MISSING.clear()
    with caplog.at_level(logging.WARNING):
        healthy({"other": torch.zeros(1)})
        healthy({"other": torch.zeros(1)})
    assert caplog.text.count("'state' was missing from the batch during normalization") == 1
