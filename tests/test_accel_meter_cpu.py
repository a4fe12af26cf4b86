"""The ``accel`` uncertainty proxy: meter arithmetic, masks from the normalisation statistics, the enable switch and
its precedence, publication by the policy wrappers (single draw and best-of-N), and the checkpoint diagnostic."""

import copy
import math

import pytest
import torch

from helpers import tiny_batch, tiny_pi05
from opentau_b200.datasets.synthetic import identity_stats
from opentau_b200.policies import accel as A
from opentau_b200.policies.candidates import configure_candidates
from opentau_b200.scripts import diagnose_accel as D


def _stats_with_padding(real: int = 7):
    s = copy.deepcopy(identity_stats())
    s["actions"]["std"][real:] = 0.0
    for k in ("min", "max", "q01", "q99"):
        if k in s["actions"]:
            s["actions"][k][real:] = 0.0
    return s


def test_meter_formula_nan_cases_and_prefix_trace():
    v = [torch.tensor([[[1.0, 0.0]]]), torch.tensor([[[1.0, 1.0]]]), torch.tensor([[[0.0, 1.0]]]),
         torch.tensor([[[5.0, 5.0]]])]
    with A.record_traces() as sink:
        m = A.AccelMeter(3, 1, torch.device("cpu"), record_trace=True)
        sink.append(m)
        for x in v:
            m.update(x)                                   # the fourth is past the prefix and ignored
    num = 1.0 + 1.0
    den = 1.0 + math.sqrt(2.0) + 1.0
    assert m.steps == 3 and m.value().item() == pytest.approx(3 * num / den)
    assert m.value_at(2).item() == pytest.approx(2 * 1.0 / (1.0 + math.sqrt(2.0)))
    assert set(m.prefix_values()) == {2, 3} and m.to_list() == [pytest.approx(3 * num / den)]
    with pytest.raises(ValueError):
        m.value_at(4)
    short = A.AccelMeter(2, 1, torch.device("cpu"))
    short.update(v[0])
    assert math.isnan(short.value().item())                # one velocity: empty numerator, not "certain"
    masked = A.AccelMeter(2, 1, torch.device("cpu"), dim_mask=torch.zeros(1, 2, dtype=torch.bool))
    masked.update(v[0]); masked.update(v[1])
    assert math.isnan(masked.value().item())               # everything masked out
    with pytest.raises(RuntimeError):
        short.value_at(2)
    with pytest.raises(ValueError):
        A.AccelMeter(1, 1, torch.device("cpu"))


def test_prefix_rules_and_row_mask():
    assert A.default_prefix(10) == 9 and A.default_prefix(2) == 2 and A.resolve_prefix(None, 10) is None
    assert A.resolve_prefix(50, 10) == 10
    with pytest.raises(ValueError):
        A.default_prefix(1)
    with pytest.raises(ValueError):
        A.resolve_prefix(1, 10)
    frozen = torch.zeros(2, 10, dtype=torch.bool)
    frozen[1, :3] = True
    rows = A.executed_row_mask(prefix_mask=frozen, delay=torch.tensor([0, 3]), chunk_size=10, n_action_steps=4,
                               device="cpu")
    assert rows[0].tolist() == [True] * 4 + [False] * 6
    assert rows[1].tolist() == [False] * 3 + [True] * 4 + [False] * 3     # [delay, delay + n_action_steps)


def test_dim_mask_and_scale_come_from_the_action_statistics():
    pol = tiny_pi05()
    pol.unnormalize_outputs = type(pol.unnormalize_outputs)(
        pol.config.output_features, pol.config.normalization_mapping,
        per_dataset_stats=[_stats_with_padding(7), _stats_with_padding(0)])
    idx = torch.tensor([0, 0])
    mask = A.resolve_action_dim_mask(pol.unnormalize_outputs, max_action_dim=32, dataset_index=idx)
    assert mask.shape == (2, 32) and mask[0, :7].all() and not mask[0, 7:].any()
    scale = A.action_dim_scale(pol.unnormalize_outputs, max_action_dim=40, dataset_index=idx)
    assert scale.shape == (2, 40) and (scale > 0).all() and (scale[:, 7:] == 1).all()
    with pytest.raises(ValueError, match=r"Head\(s\) \[0\] do have usable stats"):
        A.resolve_action_dim_mask(pol.unnormalize_outputs, max_action_dim=32, dataset_index=torch.tensor([1]))
    from opentau_b200.configs.types import NormalizationMode
    ident = type(pol.unnormalize_outputs)(pol.config.output_features, {"ACTION": NormalizationMode.IDENTITY},
                                          per_dataset_stats=[identity_stats()])
    with pytest.raises(ValueError, match="IDENTITY"):
        A.resolve_action_dim_mask(ident, max_action_dim=32, dataset_index=idx)


def test_configure_precedence_and_refusals(monkeypatch):
    pol = tiny_pi05()
    cfg = type("C", (), {"policy": type("P", (), {"accel_prefix": 4, "type": "pi05"})()})()
    monkeypatch.delenv(A.ACCEL_PREFIX_ENV, raising=False)
    assert A.configure_accel(pol, None) is None and pol.accel_prefix is None
    monkeypatch.setenv(A.ACCEL_PREFIX_ENV, "auto")
    assert A.configure_accel(pol, None) == pol.config.num_steps - 1          # environment
    assert A.configure_accel(pol, cfg) == 4                                  # config beats environment
    assert A.configure_accel(pol, cfg, override="3") == 3                    # the entry point's flag beats both
    with pytest.raises(ValueError, match="integer"):
        A.configure_accel(pol, cfg, override="soon")
    with pytest.raises(ValueError, match=">= 2"):
        A.configure_accel(pol, cfg, override=1)
    with pytest.raises(ValueError, match="not wired"):
        A.configure_accel(torch.nn.Linear(1, 1), cfg)


def test_provenance_round_trip_and_comparability():
    pol = tiny_pi05()
    pol.accel_prefix = 4
    m = A.make_meter(pol, batch_size=2, device="cpu")
    p = A.build_provenance(pol, m, dataset_index=torch.tensor([0, 0]))
    assert p.prefix == 4 and p.num_scored_dims == (32, 32) and p.velocity_dtype == "float32"
    q = A.AccelProvenance.from_dict({**p.to_dict(), "a_future_key": 1})
    assert q == p
    A.assert_comparable(p, A.AccelProvenance.from_dict({**p.to_dict(), "dataset_index": [3], "num_scored_dims": [7]}))
    with pytest.raises(ValueError, match="prefix: calibrated on 4, observed 5"):
        A.assert_comparable(p, A.AccelProvenance.from_dict({**p.to_dict(), "prefix": 5}))
    with pytest.raises(ValueError, match="n_candidates"):
        A.assert_comparable(p, A.AccelProvenance.from_dict({**p.to_dict(), "n_candidates": 4}))


def test_policy_publishes_the_score_for_single_draws_and_for_the_selected_candidate():
    pol = tiny_pi05(num_steps=5)
    b = tiny_batch(batch_size=2)
    pol.sample_actions(b)
    assert pol.last_accel is None                                  # off until armed
    A.configure_accel(pol, None, override="auto")
    a1 = pol.sample_actions(b)
    assert a1.shape == (2, 10, 32) and len(pol.last_accel) == 2 and all(math.isfinite(v) and v >= 0 for v in pol.last_accel)
    assert pol.last_accel_provenance.prefix == 4 and pol.last_accel_provenance.n_candidates == 1
    with A.record_traces() as meters:
        pol.sample_actions(b)
    assert len(meters) == 1 and set(meters[0].prefix_values()) == {2, 3, 4}
    configure_candidates(pol, 3, "medoid")
    a3 = pol.sample_actions(b)
    assert a3.shape == (2, 10, 32) and len(pol.last_accel) == 2 and len(pol.last_accel_candidates) == 2
    assert all(len(row) == 3 for row in pol.last_accel_candidates) and len(pol.last_candidate_scores[0]) == 3
    assert all(v in row for v, row in zip(pol.last_accel, pol.last_accel_candidates))
    assert pol.last_accel_provenance.n_candidates == 3
    pol.reset()
    assert pol.last_accel is None


def test_spearman_and_draw_allocation():
    assert D.spearman([1, 2, 3, 4], [10, 20, 30, 40]) == pytest.approx(1.0)
    assert D.spearman([1, 2, 3, 4], [4, 3, 2, 1]) == pytest.approx(-1.0)
    assert D.spearman([1, 2, float("nan"), 4, 5], [2, 1, 0, 4, 5]) == pytest.approx(0.8)
    assert math.isnan(D.spearman([1, 2], [2, 1])) and math.isnan(D.spearman([1, 1, 1], [1, 2, 3]))
    assert D.allocate_draws([100, 100, 100], 6) == [2, 2, 2]
    assert D.allocate_draws([100, 100, 1], 9) == [4, 4, 1]          # the short member is made up by the others
    assert D.allocate_draws([1, 100, 100], 9) == [1, 4, 4]
    assert sum(D.allocate_draws([5, 5, 5], 2)) == 2                 # fewer draws than datasets never rounds up
    assert D.allocate_draws([2, 3], 50) == [2, 3]


def test_diagnostic_report_on_a_tiny_policy():
    pol = tiny_pi05(num_steps=4)
    obs = [tiny_batch(batch_size=1, seed=s) for s in range(3)]
    rep = D.diagnose_accel(pol, obs, num_noise_repeats=2, num_resamples=2)
    assert rep.prefix == 3 and rep.num_scored_dims == [32] and len(rep.serving_scores) == 3
    assert rep.dtype_floor == pytest.approx(0.0, abs=1e-5)          # fp32 is the serving dtype on CPU
    assert set(rep.prefix_sweep) == {2, 3, 4} and rep.prefix_study.num_observations == 3
    assert set(rep.prefix_study.rho) == {2, 3, 4} and len(rep.prefix_study.divergences) == 3
    assert pol.accel_prefix == 3                                    # the study restored the prefix it widened
    text = D.format_report(rep)
    assert "accel diagnostic" in text and "prefix quality" in text and "signal / floor" in text
    import json
    json.dumps(rep.to_dict())
    assert math.isnan(D.signal_to_floor(1.0, float("nan"))) and D.signal_to_floor(1.0, 0.0) == float("inf")
    rep.signal_to_floor = float("nan")
    assert "NOT MEASURED" in D.format_report(rep)
    with pytest.raises(ValueError, match="at least two"):
        D.diagnose_accel(pol, obs[:1])


def test_candidate_configuration_rules():
    """Precedence, refusals and the critic's own requirements (reference ``src/opentau/policies/candidates.py``)."""
    from types import SimpleNamespace

    from opentau_b200.policies import candidates as C
    pol = tiny_pi05(num_steps=5)
    cfg = SimpleNamespace(policy=SimpleNamespace(n_candidates=3, action_chunk_critic_path="medoid", type="pi05"))
    assert C.configure_candidates(pol, cfg) == 3 and isinstance(pol._critic, C.MedoidCritic)
    # the critic is bound, not registered: nothing of it reaches the policy's state dict or parameters
    assert "_critic" not in dict(pol.named_children()) and not pol._critic.state_dict()
    # an entry point's override of 1 disables a config-enabled N and clears the critic
    assert C.configure_candidates(pol, cfg, override=1) == 1 and pol._critic is None and pol._n_candidates == 1
    # N > 1 without a critic path, a learned-critic path, a critic without score_chunks, a bad count
    cfg.policy.action_chunk_critic_path = None
    with pytest.raises(ValueError, match="action_chunk_critic_path"):
        C.configure_candidates(pol, cfg)
    cfg.policy.action_chunk_critic_path = "critics/v1"
    with pytest.raises(NotImplementedError, match="learned critic"):
        C.configure_candidates(pol, cfg)
    with pytest.raises(TypeError, match="score_chunks"):
        C.configure_candidates(pol, cfg, critic=object())
    with pytest.raises(ValueError, match=">= 1"):
        C.configure_candidates(pol, cfg, override=0)
    # the consensus selector cannot rank two candidates: the start-up probe says so
    with pytest.raises(ValueError, match=">= 3"):
        C.configure_candidates(pol, 2, "medoid")

    class WrongShape:
        def score_chunks(self, batch, candidates, *, row_mask, dataset_index):
            return candidates.new_zeros(candidates.shape[0])
    with pytest.raises(TypeError, match=r"\(B, N\)"):
        C.configure_candidates(pol, 3, WrongShape())
    # a family without a best-of-N sampler: silent at N == 1, refused above
    bare = SimpleNamespace(config=SimpleNamespace(max_action_dim=8))
    assert C.configure_candidates(bare, SimpleNamespace(n_candidates=1)) == 1 and not hasattr(bare, "_n_candidates")
    with pytest.raises(ValueError, match="no best-of-N sampler"):
        C.configure_candidates(bare, SimpleNamespace(n_candidates=4, type="value"))
    # entry points that cannot honour the setting
    C.refuse_candidates(SimpleNamespace(policy=SimpleNamespace(n_candidates=1)), reason="x")
    with pytest.raises(ValueError, match="not supported here: static graph"):
        C.refuse_candidates(SimpleNamespace(policy=SimpleNamespace(n_candidates=4)), reason="static graph")
    t = torch.arange(12.).view(6, 2)
    assert torch.equal(C.collapse_candidates(C.expand_candidates(t[:2], 3), 3)[1, 2], t[1])


def test_medoid_scores_in_the_policy_normalised_space():
    """A dim with a large raw scale must not dominate: the distance is taken after the policy's per-dim scale, over
    dims with a spread and executed rows only."""
    from opentau_b200.policies import candidates as C
    pol = tiny_pi05(num_steps=5)
    critic = C.load_critic("medoid", policy=pol)
    real = pol.config.action_feature.shape[0]
    scale = A.action_dim_scale(pol.unnormalize_outputs, max_action_dim=real, dataset_index=torch.zeros(1).long())[0]
    keep = A.resolve_action_dim_mask(pol.unnormalize_outputs, max_action_dim=real,
                                     dataset_index=torch.zeros(1).long())[0]
    cand = torch.randn(1, 4, pol.config.chunk_size, real)
    rows = torch.ones(1, pol.config.chunk_size, dtype=torch.bool)
    rows[:, 3:] = False
    got = critic.score_chunks({}, cand, row_mask=rows, dataset_index=torch.zeros(1).long())
    x = (cand[0, :, :3] / scale)[..., keep].flatten(1)
    want = -(torch.cdist(x, x).sum(-1) / 3)
    torch.testing.assert_close(got[0], want)
    # rows that are not executed do not matter
    cand2 = cand.clone()
    cand2[:, :, 3:] += 100.0
    torch.testing.assert_close(critic.score_chunks({}, cand2, row_mask=rows, dataset_index=torch.zeros(1).long()), got)
    with pytest.raises(ValueError, match="row_mask"):
        critic.score_chunks({}, cand, row_mask=rows[0], dataset_index=torch.zeros(1).long())
