"""Other policy families on CPU with tiny geometries: pi0, pi0.6, cosmos3 (+ layer conditioning)."""

import pytest
import torch

from helpers import TINY, tiny_batch
from opentau_b200.configs.types import FeatureType, PolicyFeature
from opentau_b200.datasets.synthetic import identity_stats
from opentau_b200.policies.factory import get_policy_class, make_policy, make_policy_config

FEATS = {"camera0": PolicyFeature(FeatureType.VISUAL, (3, 224, 224)), "state": PolicyFeature(FeatureType.STATE, (32,))}
OUT = {"actions": PolicyFeature(FeatureType.ACTION, (32,))}


def _pi06():
    return make_policy_config(
        "pi06", chunk_size=10, n_action_steps=10, prompt_max_length=16, discrete_action_max_length=8,
        discrete_action_vocab_size=256, dropout=0.0, device="cpu", resize_imgs_with_padding=(224, 224),
        input_features=dict(FEATS), output_features=dict(OUT),
        vlm=dict(TINY["vlm"], num_key_value_heads=2, sliding_window_pattern=2),
        expert=dict(TINY["expert"], num_key_value_heads=2), vision=TINY["vision"],
        vlm_config={"tokens_per_image_side": 8})


def _pi0(**kw):
    return make_policy_config("pi0", chunk_size=10, n_action_steps=10, tokenizer_max_length=16, dropout=0.0,
                              device="cpu", input_features=dict(FEATS), output_features=dict(OUT), **TINY, **kw)


def _cosmos3(col=None, layers=3):
    return make_policy_config(
        "cosmos3", chunk_size=10, n_action_steps=10, prompt_max_length=16, dropout=0.0, device="cpu",
        image_resize=128, input_features=dict(FEATS), output_features=dict(OUT), num_steps=3,
        backbone=dict(hidden_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                      intermediate_size=256, vocab_size=1024, mrope_sections=(6, 5, 5)),
        vision=dict(hidden_size=64, depth=3, num_heads=4, intermediate_size=128, num_position_embeddings=64,
                    deepstack_visual_indexes=(0, 1)),
        expert_hidden_size=64, expert_intermediate_size=128, expert_num_hidden_layers=layers,
        expert_num_attention_heads=4, expert_num_key_value_heads=2, expert_head_dim=32, expert_adarms_cond_dim=32,
        proj_width=64, condition_on_layer=col)


@pytest.mark.parametrize("builder", [_pi06, _pi0, _cosmos3])
def test_forward_backward_sample(builder):
    torch.manual_seed(0)
    pol = make_policy(builder(), per_dataset_stats=[identity_stats()])
    b = tiny_batch()
    out = pol(b)
    assert set(out) >= {"MSE", "CE"} and torch.isfinite(out["MSE"])
    (out["MSE"] + out["CE"]).backward()
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in pol.parameters() if p.requires_grad)
    pol.eval()
    a = pol.sample_actions(b)
    assert a.shape == (4, 10, 32) and torch.isfinite(a).all()
    assert pol.select_action(b).shape == (4, 32)


def test_pi06_layout_and_keys():
    pol = make_policy(_pi06(), per_dataset_stats=[identity_stats()])
    b = tiny_batch()
    images, masks = pol.prepare_images(b)
    embs, pad, att, _ = pol.model.embed_prefix(images, masks, b["lang_tokens"], b["lang_masks"], None, None,
                                               b["discrete_actions"], b["discrete_action_masks"])
    assert embs.shape[1] == 64 + 16 + 8            # pooled image tokens + causal prompt + FAST tokens (no indicator)
    assert att[0, :64].sum() == 0 and att[0, 64:].all()
    keys = set(pol.state_dict())
    pre = "model.gemma3_with_expert."
    for k in (pre + "interleaved_layers.0.backbone_layer.self_attn.q_norm.weight",
              pre + "interleaved_layers.1.backbone_layer.pre_feedforward_layernorm.weight",
              pre + "interleaved_layers.0.expert_layer.input_layernorm.dense.weight",
              pre + "gemma3.model.multi_modal_projector.mm_input_projection_weight",
              pre + "gemma3.model.language_model.embed_tokens.weight", pre + "gemma_expert.model.norm.dense.bias"):
        assert k in keys, k
    cfg = pol.model.wrapper.vlm_cfg
    assert cfg.layer_theta(0) == 10_000.0 and cfg.layer_theta(1) == 1_000_000.0


def test_pi0_trains_vlm_jointly_and_awr_weights_loss():
    torch.manual_seed(0)
    pol = make_policy(_pi0(use_awr=True), per_dataset_stats=[identity_stats()])
    b = tiny_batch()
    noise, time = torch.randn(4, 10, 32), torch.full((4,), 0.5)
    base = pol(b, noise=noise, time=time)["MSE"]
    b["advantage"] = torch.full((4,), 1.0)
    weighted = pol(b, noise=noise, time=time)["MSE"]
    torch.testing.assert_close(weighted, base * torch.e, rtol=1e-4, atol=1e-5)
    weighted.backward()
    vlm = pol.model.wrapper.paligemma.language_model
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in vlm.layers[0].parameters())
    names = {n for n, _ in pol.named_parameters()}
    assert "model.action_time_mlp_in.weight" in names and "model.time_mlp_in.weight" not in names
    b2 = {k: v for k, v in b.items() if k not in ("lang_tokens", "lang_masks")}
    b2["prompt"] = ["pick up the cube"] * 4
    assert torch.isfinite(pol(b2)["MSE"])


def test_cosmos3_backbone_is_frozen_and_layer_conditioning_truncates():
    pol = make_policy(_cosmos3(), per_dataset_stats=[identity_stats()])
    assert all(not p.requires_grad for p in pol.model.qwen3vl_with_expert.backbone.parameters())
    assert all(n.startswith("model.") and "backbone" not in n for n, p in pol.named_parameters() if p.requires_grad)
    pol2 = make_policy(_cosmos3(col=1, layers=5), per_dataset_stats=[identity_stats()])
    w = pol2.model.qwen3vl_with_expert
    assert len(w.backbone.language_model.layers) == 2 and len(w.expert.layers) == 5
    with pytest.raises(ValueError):
        make_policy(_cosmos3(col=None, layers=5), per_dataset_stats=[identity_stats()])
    keys = set(pol.state_dict())
    for k in ("model.qwen3vl_with_expert.expert.layers.0.self_attn.q_norm.weight",
              "model.qwen3vl_with_expert.expert.norm.dense.weight",
              "model.qwen3vl_with_expert.backbone.model.language_model.layers.0.self_attn.k_proj.weight",
              "model.qwen3vl_with_expert.backbone.model.visual.blocks.0.attn.qkv.weight", "model.adarms_proj.weight"):
        assert k in keys, k


def test_factory_registry():
    for name in ("pi0", "pi05", "pi06", "cosmos3", "cosmos3_nano"):
        assert get_policy_class(name).name == name
    with pytest.raises(NotImplementedError):
        get_policy_class("nope")


def test_policy_level_freeze_flags():
    """The "train only ..." flags reach the projections on the flow-matching module, not just the wrapper."""
    from opentau_b200.policies.utils import (freeze_policy_level_params_for_state_action_representation_only,
                                             freeze_policy_level_params_for_vision_only)

    from helpers import tiny_pi05_config as _pi05

    pol = make_policy(_pi05(train_vision_encoder_only=True, freeze_vision_encoder=False, train_expert_only=False), per_dataset_stats=[identity_stats()])
    names = {n for n, p in pol.model.named_parameters() if p.requires_grad}
    assert names and all("vision_tower" in n or "multi_modal_projector" in n for n in names)

    pol = make_policy(_pi05(train_state_action_representation_only=True, train_expert_only=False), per_dataset_stats=[identity_stats()])
    names = {n for n, p in pol.model.named_parameters() if p.requires_grad}
    heads = {n.split(".")[-2] for n in names}
    assert heads - {"state_proj"} == {"action_in_proj", "action_out_proj", "discrete_action_embedding", "da_head"}
    pol.train()
    w = pol.model.wrapper
    assert not w.paligemma.training and w.da_head.training          # the frozen trunk stays in eval mode

    class Outer(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.inner = torch.nn.Linear(2, 2)
            self.state_proj = torch.nn.Linear(2, 2)
            self.time_mlp_in = torch.nn.Linear(2, 2)
            self.video = torch.nn.Module()
            self.video.motion_module = torch.nn.Linear(2, 2)

    o = Outer()
    freeze_policy_level_params_for_vision_only(o, o.inner)
    assert {n for n, p in o.named_parameters() if p.requires_grad} == {
        "inner.weight", "inner.bias", "video.motion_module.weight", "video.motion_module.bias"}
    o = Outer()
    left = freeze_policy_level_params_for_state_action_representation_only(o, o.inner)
    assert left == ["state_proj.bias", "state_proj.weight"] and not o.video.motion_module.weight.requires_grad
    assert o.inner.weight.requires_grad            # the wrapper's own parameters are not touched here
