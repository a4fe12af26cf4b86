"""Response generation at inference: greedy decoding behind the cached prefix equals the teacher-forced full pass."""

import torch

from helpers import tiny_batch, tiny_pi05
from opentau_b200 import ops


def _policy(**over):
    return tiny_pi05(predict_response=True, response_max_length=6, **over).eval()


def test_generated_tokens_match_a_full_pass_over_the_same_text():
    pol = _policy()
    model, cfg = pol.model, pol.config
    b = tiny_batch()
    B = b["state"].shape[0]
    torch.manual_seed(0)
    noise = torch.randn(B, cfg.chunk_size, cfg.max_action_dim)
    actions = pol.sample_actions(b, noise=noise)
    toks, masks = model.last_response_tokens, model.last_response_masks
    tok = pol.language_tokenizer
    assert toks.shape == (B, 6) and bool((toks[:, 0] == tok.bos_token_id).all()) and bool(masks[:, 0].all())
    assert isinstance(pol.last_response, list) and len(pol.last_response) == B
    # teacher forcing: one pass over prefix + the generated tokens; the output at token i predicts token i + 1
    idx = pol._resolve_dataset_index(b, B, b["state"].device)
    nb = pol.normalize_inputs(b, idx)
    images, img_masks = pol.prepare_images(nb)
    lang_tokens, lang_masks = pol.prepare_language(nb)
    embs, pad, att, pos = model.embed_prefix(images, img_masks, lang_tokens, lang_masks, response_tokens=toks,
                                             response_masks=masks)
    blk, valid = ops.make_block_ids(pad, att)
    if pos is None:
        pos = torch.cumsum(pad, dim=1) - 1
    with torch.no_grad():
        (out, _), _ = model.wrapper(inputs_embeds=[embs, None], position_ids=pos, q_blk=blk, q_valid=valid)
    logits = ops.linear(out[:, -6:], model.wrapper.lm_head_weight()).float()
    predicted = logits.argmax(-1)
    for i in range(5):
        live = masks[:, i + 1]
        assert torch.equal(predicted[:, i][live], toks[:, i + 1][live]), i
    # after <eos> a sample only pads, and pads are neither attended nor counted as positions
    done = ((toks == tok.eos_token_id) | (toks == tok.pad_token_id)).cumsum(1) > 0
    assert bool((~masks[:, 2:] | ~done[:, :-2][:, :masks.shape[1] - 2]).all())
    assert torch.isfinite(actions).all()


def test_response_is_shared_by_candidates_and_skipped_when_off():
    pol = _policy()
    b = tiny_batch()
    B = b["state"].shape[0]
    pol.sample_actions(b)
    one = pol.model.last_response_tokens.clone()
    out = pol.sample_actions(b, n_candidates=3)
    assert out.shape[0] == B and torch.equal(pol.model.last_response_tokens, one)      # greedy: independent of the noise
    off = tiny_pi05().eval()
    off.sample_actions(b)
    assert off.last_response is None and off.model.last_response_tokens is None


def test_an_early_eos_pads_the_rest():
    pol = _policy()
    model = pol.model
    tok = pol.language_tokenizer
    head = model.wrapper.lm_head_weight()
    # make <eos> the arg-max whatever the input: every sample stops after <bos>, <eos>
    with torch.no_grad():
        head.zero_()
        head[tok.eos_token_id] = 0.0
    b = tiny_batch()
    pol.sample_actions(b)
    toks, masks = model.last_response_tokens, model.last_response_masks
    # an all-zero head gives equal logits: arg-max is id 0 = pad, which ends the sample just like <eos>
    assert bool((toks[:, 0] == tok.bos_token_id).all())
    assert bool((toks[:, 2:] == tok.pad_token_id).all()) and not bool(masks[:, 2:].any())
