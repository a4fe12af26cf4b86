"""pi0.5-MEM: STSS local correlation against the global-correlation definition, zero-initialised motion residual,
MRoPE prefix positions, training / sampling with both video encoders, rolling history at inference."""

import pytest
import torch

from helpers import TINY, tiny_batch
from opentau_b200.configs.types import FeatureType, PolicyFeature
from opentau_b200.datasets.synthetic import identity_stats
from opentau_b200.models.motion_module import MotionModule, STSSTransformation, local_correlation
from opentau_b200.policies.factory import make_policy, make_policy_config
from opentau_b200.policies.pi05_mem.modeling_pi05_mem import build_mrope_prefix_positions


def test_local_correlation_equals_windowed_global_correlation():
    torch.manual_seed(0)
    a, b = torch.randn(2, 6, 5, 7), torch.randn(2, 6, 5, 7)
    k, d = 3, 1
    got = local_correlation(a, b, k, "cosine")
    an, bn = torch.nn.functional.normalize(a, dim=1), torch.nn.functional.normalize(b, dim=1)
    glob = torch.einsum("bchw,bcuv->bhwuv", an, bn)
    want = torch.zeros(2, 5, 7, k, k)
    for h in range(5):
        for w in range(7):
            for u in range(k):
                for v in range(k):
                    hh, ww = h + u - d, w + v - d
                    if 0 <= hh < 5 and 0 <= ww < 7:
                        want[:, h, w, u, v] = glob[:, h, w, hh, ww]
    assert torch.allclose(got, want, atol=1e-6)
    sm = local_correlation(a, b, k, "dotproduct_softmax")
    assert torch.allclose(sm.flatten(-2).sum(-1), torch.ones(2, 5, 7), atol=1e-5) and float(sm[0, 0, 0, 0, 0]) == 0.0


def test_temporal_window_clamps_at_the_ends():
    t, h, w, C = 4, 3, 3, 8
    x = torch.randn(1 * t * h * w, C)
    s = STSSTransformation((3, 3, 3))(x, t, h, w)
    assert s.shape == (1, t, h, w, 3, 3, 3)
    # offset 0 (middle of the window) correlates a frame with itself: centre similarity is 1
    assert torch.allclose(s[0, :, :, :, 1, 1, 1], torch.ones(t, h, w), atol=1e-5)
    # at t=0 the "previous" frame is frame 0 itself (clamped)
    assert torch.allclose(s[0, 0, :, :, 0], s[0, 0, :, :, 1], atol=1e-6)


def test_window_correlation_over_token_major_features_matches_the_two_tensor_form():
    """The op the motion module calls (token-major features, all frame offsets at once) against ``local_correlation``
    applied frame pair by frame pair, for every correlation variant, L = 1 included, on a non-square grid."""
    from opentau_b200.ops.stss import local_window_correlation, target_frames
    torch.manual_seed(1)
    B, t, h, w, C = 2, 4, 3, 5, 8
    x = torch.randn(B * t * h * w, C)
    for L, k in ((3, 3), (1, 3), (5, 5)):
        idx = target_frames(t, L, "cpu")
        assert idx.shape == (t, L) and int(idx.min()) == 0 and int(idx.max()) <= t - 1
        for func in ("cosine", "dotproduct", "dotproduct_softmax"):
            got = STSSTransformation((L, k, k), func)(x, t, h, w)
            v = x.view(B, t, h, w, C).permute(0, 1, 4, 2, 3)
            for ti in range(t):
                for li in range(L):
                    want = local_correlation(v[:, ti], v[:, int(idx[ti, li])], k, func)
                    assert torch.allclose(got[:, ti, :, :, li], want, atol=1e-5), (L, k, func, ti, li)
    raw = local_window_correlation(x.view(B, t, h * w, C), t, h, w, 3, 3)
    assert raw.shape == (B, t, h * w, 3, 9)
    with pytest.raises(ValueError):
        local_window_correlation(x.view(B, t, h * w, C), t, h, w, 2, 3)


def test_motion_module_is_a_noop_at_init_and_learns():
    torch.manual_seed(0)
    mm = MotionModule(32, 16, 32, window=(3, 3, 3), ext_chnls=(8,), int_chnls=(8, 8, 12))
    x = torch.randn(2 * 3 * 4 * 4, 32)
    grid = torch.tensor([[3, 4, 4]] * 2)
    assert float(mm(x, grid).abs().max()) == 0.0
    keys = set(mm.state_dict())
    assert {"stss_encoders.0.stss_extraction.conv0.0.weight", "stss_encoders.0.stss_extraction.conv0.1.weight",
            "stss_encoders.0.stss_integration.fuse.1.weight", "stss_encoders.0.ln_pre.weight", "out_proj.weight"} <= keys
    assert mm.state_dict()["stss_encoders.0.stss_extraction.conv0.0.weight"].shape == (8, 9, 1, 1, 1)
    assert mm.state_dict()["stss_encoders.0.stss_integration.fuse.1.weight"].shape == (12, 8 * 3, 1, 1, 1)
    mm.out_proj.weight.data.normal_(0, 0.02)
    out = mm(x, grid)
    out.sum().backward()
    assert out.shape == (96, 32) and mm.stss_encoders[0].in_proj.weight.grad.abs().sum() > 0
    full = MotionModule(32, 16, 32, window=(3, 3, 3), ext_chnls=(8,), int_chnls=(8, 8, 12), int_mode="full",
                        zero_init_residual=False)
    assert full(x, grid).shape == (96, 32)


def test_mrope_prefix_positions():
    vid = torch.tensor([[True] * 4, [False] * 4])           # sample 1 has no camera
    txt = torch.tensor([[True, True, False], [True, True, True]])
    pos = build_mrope_prefix_positions([vid, txt], [True, False], grid=2)
    assert pos.shape == (3, 2, 7)
    assert pos[0, 0, :4].tolist() == [0, 0, 0, 0] and pos[1, 0, :4].tolist() == [0, 0, 1, 1] and pos[2, 0, :4].tolist() == [0, 1, 0, 1]
    assert pos[:, 0, 4:].tolist() == [[2, 3, 3]] * 3          # text resumes after `grid` units
    assert pos[:, 1, 4:].tolist() == [[0, 1, 2]] * 3          # absent video advances nothing


def _cfg(**kw):
    feats = {"camera0": PolicyFeature(FeatureType.VISUAL, (3, 224, 224)), "state": PolicyFeature(FeatureType.STATE, (32,))}
    base = dict(chunk_size=10, n_action_steps=10, prompt_max_length=16, discrete_action_max_length=8,
                discrete_action_vocab_size=256, dropout=0.0, device="cpu", n_obs_steps=3, spacetime_layer_stride=2,
                input_features=feats, output_features={"actions": PolicyFeature(FeatureType.ACTION, (32,))},
                motion_window=(3, 5, 5), motion_hidden_dim=16, motion_insert_layer=0, **TINY)
    return make_policy_config("pi05_mem", **{**base, **kw})


def _hist_batch(B=2, T=3):
    b = tiny_batch(batch_size=B)
    b["camera0"] = torch.rand(B, T, 3, 224, 224)
    b["state"] = torch.randn(B, T, 32) * 0.3
    b["obs_history_is_pad"] = torch.tensor([[True, False, False], [False, False, False]])[:B]
    return b


@pytest.mark.parametrize("use_motion,rope", [(False, "mrope_interleaved"), (True, "mrope_interleaved"), (False, "rope")])
def test_train_and_sample(use_motion, rope):
    torch.manual_seed(0)
    pol = make_policy(_cfg(use_motion=use_motion, rope_type=rope), per_dataset_stats=[identity_stats()])
    b = _hist_batch()
    out = pol(b)
    assert torch.isfinite(out["MSE"]) and torch.isfinite(out["CE"])
    (out["MSE"] + out["CE"]).backward()
    assert pol.model.state_proj.weight.grad.abs().sum() > 0
    if use_motion:
        assert any(k.startswith("model.video_encoder.motion_module.") for k in pol.state_dict())
        assert pol.model.video_encoder.motion_module.out_proj.weight.grad is not None
    assert not any("video_encoder.vision" in k for k in pol.state_dict())      # the tower is stored once
    pol.eval()
    a = pol.sample_actions(b)
    assert a.shape == (2, 10, 32) and torch.isfinite(a).all()


def test_padded_history_does_not_change_the_result():
    """A frame flagged as padding must be invisible: changing its pixels and state changes nothing."""
    torch.manual_seed(0)
    pol = make_policy(_cfg(), per_dataset_stats=[identity_stats()]).eval()
    b = _hist_batch()
    noise = torch.randn(2, 10, 32)
    a1 = pol.sample_actions(b, noise=noise)
    b2 = dict(b)
    b2["camera0"] = b["camera0"].clone()
    b2["camera0"][0, 0] = torch.rand(3, 224, 224)
    b2["state"] = b["state"].clone()
    b2["state"][0, 0] = 5.0
    a2 = pol.sample_actions(b2, noise=noise)
    assert torch.allclose(a1, a2, atol=1e-5)


def test_rolling_history_at_inference():
    pol = make_policy(_cfg(n_action_steps=1), per_dataset_stats=[identity_stats()]).eval()
    pol.reset()
    one = tiny_batch(batch_size=1)
    hb = pol._build_history_batch(one)
    assert hb["camera0"].shape == (1, 3, 3, 224, 224) and hb["obs_history_is_pad"].tolist() == [[True, True, False]]
    hb = pol._build_history_batch(one)
    assert hb["obs_history_is_pad"].tolist() == [[True, False, False]]
    pol.reset()
    assert pol.select_action(one).shape == (1, 32)
