"""Tiny pi0.5 on CPU: layout, losses, knowledge insulation, sampling, checkpoint key names."""

import torch

from helpers import tiny_batch, tiny_pi05, tiny_pi05_config


def test_forward_returns_loss_dict_and_all_trainable_params_get_grads():
    pol = tiny_pi05()
    out = pol(tiny_batch())
    assert set(out) == {"MSE", "CE"}
    (out["MSE"] + out["CE"]).backward()
    missing = [n for n, p in pol.named_parameters() if p.requires_grad and p.grad is None]
    assert missing == []
    frozen = [n for n, p in pol.named_parameters() if not p.requires_grad]
    assert any("vision_tower" in n for n in frozen)


def test_prefix_layout_lengths():
    pol = tiny_pi05()
    b = tiny_batch()
    m = pol.model
    images, masks = pol.prepare_images(b)
    embs, pad, att, seg = m.embed_prefix(images, masks, b["lang_tokens"], b["lang_masks"], None, None,
                                         b["discrete_actions"], b["discrete_action_masks"])
    n_img = 256
    assert embs.shape[1] == n_img + 16 + 3 + 8          # image + prompt + "Action: " indicator + FAST tokens
    assert att[0, : n_img + 16].sum() == 0              # image + language form one bidirectional block
    assert att[0, n_img + 16:].all()                    # indicator and action tokens are causal
    embs2, pad2, att2, _ = m.embed_prefix(images, masks, b["lang_tokens"], b["lang_masks"])
    assert embs2.shape[1] == n_img + 16                 # inference prefix has no discrete-action block


def test_knowledge_insulation_blocks_mse_gradient_into_vlm():
    pol = tiny_pi05(knowledge_insulation=True)
    out = pol(tiny_batch())
    out["MSE"].backward()
    vlm = pol.model.paligemma_with_expert.paligemma.language_model
    assert all(p.grad is None or p.grad.abs().sum() == 0 for p in vlm.parameters())
    expert = pol.model.paligemma_with_expert.gemma_expert
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in expert.parameters())
    pol2 = tiny_pi05(knowledge_insulation=False)
    for n, p in pol2.named_parameters():      # adaptive-norm gates are zero at init: open them
        if ".dense." in n:
            torch.nn.init.normal_(p, std=0.2)
    out2 = pol2(tiny_batch())
    out2["MSE"].backward()
    vlm2 = pol2.model.paligemma_with_expert.paligemma.language_model
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in vlm2.layers.parameters())


def test_ce_gradient_does_not_reach_expert():
    pol = tiny_pi05()
    out = pol(tiny_batch())
    out["CE"].backward()
    expert = pol.model.paligemma_with_expert.gemma_expert
    assert all(p.grad is None or p.grad.abs().sum() == 0 for p in expert.parameters())


def test_losses_are_deterministic_given_noise_and_time():
    pol = tiny_pi05()
    b = tiny_batch()
    noise = torch.randn(4, 10, 32)
    time = torch.full((4,), 0.3)
    a = pol(b, noise=noise, time=time)
    c = pol(b, noise=noise, time=time)
    assert torch.equal(a["MSE"], c["MSE"]) and torch.equal(a["CE"], c["CE"])


def test_fused_path_matches_oracle_path(monkeypatch):
    pol = tiny_pi05()
    b = tiny_batch()
    noise = torch.randn(4, 10, 32)
    time = torch.full((4,), 0.5)
    a = pol(b, noise=noise, time=time)
    (a["MSE"] + a["CE"]).backward()
    g_fused = {n: p.grad.clone() for n, p in pol.named_parameters() if p.grad is not None}
    pol.zero_grad()
    monkeypatch.setenv("OPENTAU_B200_ORACLE", "1")
    c = pol(b, noise=noise, time=time)
    (c["MSE"] + c["CE"]).backward()
    torch.testing.assert_close(a["MSE"], c["MSE"], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(a["CE"], c["CE"], rtol=1e-4, atol=1e-5)
    for n, p in pol.named_parameters():
        if p.grad is not None:
            torch.testing.assert_close(g_fused[n], p.grad, rtol=2e-3, atol=2e-5, msg=lambda m, n=n: f"{n}: {m}")


def test_sample_actions_shape_determinism_and_cache_equivalence():
    pol = tiny_pi05().eval()
    b = tiny_batch()
    noise = torch.randn(4, 10, 32)
    a1 = pol.sample_actions(b, noise=noise)
    a2 = pol.sample_actions(b, noise=noise)
    assert a1.shape == (4, 10, 32)
    assert torch.equal(a1, a2)
    # one denoise step against the cache == joint forward over [prefix | suffix] without a cache
    m = pol.model
    images, masks = pol.prepare_images(b)
    cache, plen = m.prefill(images, masks, b["lang_tokens"], b["lang_masks"])
    t = torch.full((4, 10), 0.7)
    v_cached = m.denoise_step(cache, plen, noise, t)
    from opentau_b200 import ops
    pe, pp, pa, _ = m.embed_prefix(images, masks, b["lang_tokens"], b["lang_masks"])
    se, sp, sa, cond = m.embed_suffix(noise, t)
    pad = torch.cat([pp, sp], 1)
    att = torch.cat([pa, sa], 1)
    blk, valid = ops.make_block_ids(pad, att)
    pos = torch.cumsum(pad, 1) - 1
    (_, so), _ = m.paligemma_with_expert(inputs_embeds=[pe, se], position_ids=pos, q_blk=blk, q_valid=valid,
                                         adarms_cond=[None, cond])
    v_joint = m.action_out_proj(so[:, -10:]).float()
    torch.testing.assert_close(v_cached, v_joint, rtol=1e-4, atol=1e-5)


def test_best_of_n_widens_batch_and_requires_matching_noise():
    pol = tiny_pi05().eval()
    b = tiny_batch()
    m = pol.model
    images, masks = pol.prepare_images(b)
    import pytest
    with pytest.raises(ValueError):
        m.sample_actions(images, masks, b["lang_tokens"], b["lang_masks"], noise=torch.randn(4, 10, 32), n_candidates=2)
    out = m.sample_actions(images, masks, b["lang_tokens"], b["lang_masks"], noise=torch.randn(8, 10, 32),
                           n_candidates=2)
    assert out.shape == (8, 10, 32)


def test_select_action_queue():
    pol = tiny_pi05(n_action_steps=5).eval()
    b = tiny_batch()
    pol.reset()
    a = pol.select_action(b)
    assert a.shape == (4, 32)
    assert len(pol._action_queue) == 4
    for _ in range(4):
        pol.select_action(b)
    assert len(pol._action_queue) == 0


def test_state_dict_uses_reference_key_names_and_roundtrips(tmp_path):
    pol = tiny_pi05()
    keys = set(pol.state_dict().keys())
    pre = "model.paligemma_with_expert."
    for k in [pre + "paligemma.model.language_model.layers.0.self_attn.q_proj.weight",
              pre + "paligemma.model.language_model.layers.0.self_attn.k_proj.weight",
              pre + "paligemma.model.language_model.layers.0.mlp.gate_proj.weight",
              pre + "paligemma.model.language_model.layers.1.mlp.up_proj.weight",
              pre + "paligemma.model.vision_tower.vision_model.encoder.layers.0.self_attn.out_proj.bias",
              pre + "paligemma.model.vision_tower.vision_model.embeddings.patch_embedding.weight",
              pre + "paligemma.model.multi_modal_projector.linear.weight",
              pre + "gemma_expert.model.layers.0.input_layernorm.dense.weight",
              pre + "gemma_expert.model.norm.dense.bias",
              pre + "discrete_action_embedding.weight", pre + "da_head.bias",
              "model.action_in_proj.weight", "model.time_mlp_out.bias",
              "normalize_inputs.buffer_state.min", "unnormalize_outputs.buffer_actions.std"]:
        assert k in keys, k
    assert not any("qkv_proj" in k or "gate_up_proj" in k for k in keys)
    pol.save_pretrained(tmp_path / "ckpt")
    assert (tmp_path / "ckpt" / "config.json").exists() and (tmp_path / "ckpt" / "model.safetensors").exists()
    from opentau_b200.policies.pi05.modeling_pi05 import PI05Policy
    pol2 = PI05Policy.from_pretrained(tmp_path / "ckpt")
    b = tiny_batch()
    noise, time = torch.randn(4, 10, 32), torch.full((4,), 0.4)
    pol.eval()
    a, c = pol(b, noise=noise, time=time), pol2(b, noise=noise, time=time)
    torch.testing.assert_close(a["MSE"], c["MSE"])
    torch.testing.assert_close(a["CE"], c["CE"])


def test_bf16_cast_keeps_fp32_islands():
    pol = tiny_pi05().to(torch.bfloat16)
    emb = pol.model.paligemma_with_expert.paligemma.vision_tower.vision_model.embeddings
    assert emb.patch_embedding.weight.dtype == torch.float32
    assert emb.position_embedding.weight.dtype == torch.float32
    assert pol.normalize_inputs.buffer_state["min"].dtype == torch.float32
    assert pol.model.action_in_proj.weight.dtype == torch.bfloat16


def test_config_validation():
    import pytest
    with pytest.raises(ValueError):
        tiny_pi05_config(n_action_steps=20)          # > chunk_size
    with pytest.raises(ValueError):
        tiny_pi05_config(train_expert_only=True, freeze_vision_encoder=False)
    with pytest.raises(ValueError):
        tiny_pi05_config(state_type="weird")


def test_stacked_adaptive_norm_weights_follow_in_place_updates():
    """At inference the adaptive-norm projections live in one stacked buffer: sampling does not concatenate per step,
    and weights loaded afterwards are seen (no stale copy)."""
    import torch
    from helpers import tiny_batch, tiny_pi05
    pol = tiny_pi05(num_steps=2).eval()
    b = tiny_batch(batch_size=2)
    noise = torch.randn(2, 10, 32)
    a1 = pol.sample_actions(b, noise=noise)
    tower = pol.model.wrapper.decoder.towers[1]
    stack = tower._ada_stack
    first = tower.layers[0].input_layernorm.dense.weight
    assert first.data_ptr() == stack[0].data_ptr()                     # a view of the stack, not a copy
    assert torch.equal(pol.sample_actions(b, noise=noise), a1) and tower._ada_stack is stack
    sd = {k: v.clone() for k, v in pol.state_dict().items()}
    for k in sd:
        if "layernorm.dense.weight" in k:
            sd[k] = sd[k] + 0.05
    pol.load_state_dict(sd)
    a2 = pol.sample_actions(b, noise=noise)
    assert tower._ada_stack is stack and not torch.allclose(a1, a2)     # in-place load wrote through the views
    out = pol.train()(b)                                                # training still reaches the individual parameters
    (out["MSE"] + out["CE"]).backward()
    assert first.grad is not None and first.grad.abs().sum() > 0
