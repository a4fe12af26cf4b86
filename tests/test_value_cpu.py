"""Value model on CPU: return bins, expected value, losses on robot vs language-only samples, keys."""

import torch

from helpers import TINY, tiny_batch
from opentau_b200.configs.types import FeatureType, PolicyFeature
from opentau_b200.datasets.synthetic import identity_stats
from opentau_b200.policies.factory import make_policy, make_policy_config
from opentau_b200.policies.value.reward import calculate_n_step_return, calculate_return_bins_with_equal_width


def _cfg(**kw):
    feats = {"camera0": PolicyFeature(FeatureType.VISUAL, (3, 224, 224)), "state": PolicyFeature(FeatureType.STATE, (32,))}
    return make_policy_config(
        "value", prompt_max_length=16, response_max_length=6, device="cpu", input_features=feats,
        vlm=dict(TINY["vlm"], sliding_window_pattern=2), vision=TINY["vision"], **kw)


def _batch(B=4):
    b = tiny_batch(batch_size=B)
    b["return_bin_idx"] = torch.tensor([0, 50, 100, 200])[:B]
    b["return_continuous"] = torch.tensor([-1.0, -0.75, -0.5, 0.0])[:B]
    b["response"] = ["pick the cup", "", "move left", "done"][:B]
    return b


def test_return_bins():
    # episode_end_idx is exclusive: the last step of a successful episode has return 0 -> top bin
    assert calculate_return_bins_with_equal_width(True, 201, 100, 400, 99) == (200, 0.0)
    idx, r = calculate_return_bins_with_equal_width(True, 201, 100, 400, 0)
    assert r == -99 / 400 and idx == int((r + 1) * 200)
    idx_f, r_f = calculate_return_bins_with_equal_width(False, 201, 100, 400, 99, c_neg=-300.0)
    assert r_f == -0.75 and idx_f == 50
    assert calculate_n_step_return(True, 50, 100, 400, 0) == -50 / 400
    assert calculate_n_step_return(True, 50, 100, 400, 90) == -9 / 400
    assert calculate_n_step_return(False, 50, 100, 400, 0, c_neg=-100.0) == -50 / 400        # end outside window
    assert calculate_n_step_return(False, 50, 100, 400, 60, c_neg=-100.0) == (-39 - 100) / 400


def test_expected_value_from_bins():
    pol = make_policy(_cfg(), per_dataset_stats=[identity_stats()])
    n = pol.config.reward_config.number_of_bins
    logits = torch.full((2, n), -1e4)
    logits[0, 0], logits[1, -1] = 0.0, 0.0
    v = pol.calculate_value(logits)
    c = pol.bin_centres("cpu")
    assert torch.allclose(v, torch.stack([c[0], c[-1]]), atol=1e-6)
    assert -1.0 <= float(c[0]) < float(c[-1]) <= 0.0
    assert abs(float(pol.calculate_value(torch.zeros(1, n))) - float(c.mean())) < 1e-6


def test_losses_and_language_only_samples():
    torch.manual_seed(0)
    pol = make_policy(_cfg(), per_dataset_stats=[identity_stats()])
    b = _batch()
    b["action_is_pad"] = torch.zeros(4, 10, dtype=torch.bool)
    b["action_is_pad"][1] = True                       # sample 1 is a language-only (VQA) sample
    out = pol(b, return_per_sample=True)
    assert set(out) >= {"MSE", "CE", "L1", "Accuracy"} and float(out["MSE"]) == 0.0
    s, c = out["CE_per_sample"]
    # robot samples contribute exactly one value slot; the language sample contributes its response tokens
    assert c[0] == 1 and c[2] == 1 and c[3] == 1
    assert torch.isfinite(out["CE"]) and 0.0 <= float(out["Accuracy"]) <= 1.0
    out["CE"].backward()
    m = pol.model.siglip_gemma_value
    assert m.value_head.weight.grad.abs().sum() > 0 and m.value_token.grad.abs().sum() > 0
    v = pol.predict_value(b)
    assert v.shape == (4,) and ((v <= 0) & (v >= -1)).all()


def test_value_read_position_ignores_response():
    """The value token attends only to images+prompt, so the response cannot change the value logits."""
    torch.manual_seed(0)
    pol = make_policy(_cfg(), per_dataset_stats=[identity_stats()]).eval()
    b = _batch()
    nb = pol.normalize_inputs(b, torch.zeros(4, dtype=torch.long))
    images, masks = pol.prepare_images(nb)
    lt, lm = pol.prepare_language(nb)
    rt, rm = pol.prepare_response(b)
    with torch.no_grad():
        a, _ = pol.model(images, masks, lt, lm, rt, rm)
        c = pol.model.get_value(images, masks, lt, lm)
    assert torch.allclose(a, c, atol=1e-5)


def test_state_dict_keys_follow_reference_layout():
    pol = make_policy(_cfg(), per_dataset_stats=[identity_stats()])
    keys = set(pol.state_dict())
    for k in ("model.siglip_gemma_value.value_token", "model.siglip_gemma_value.value_head.weight",
              "model.siglip_gemma_value.response_head.weight", "model.state_proj.weight",
              "model.multi_modal_proj.bias", "model.siglip_gemma_value.gemma.embed_tokens.weight",
              "model.siglip_gemma_value.gemma.layers.0.self_attn.q_proj.weight",
              "model.siglip_gemma_value.gemma.layers.1.mlp.gate_proj.weight",
              "model.siglip_gemma_value.vision_encoder.vision_model.encoder.layers.0.self_attn.k_proj.weight"):
        assert k in keys, k
