"""pi0.7 controller / planner, the SpaceTime video encoder and the rank-wide branch decisions."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import TINY, tiny_batch, free_port
from opentau_b200.configs.types import FeatureType, PolicyFeature
from opentau_b200.datasets.synthetic import identity_stats
from opentau_b200.models.video_encoder import build_temporal_sinusoidal_pe
from opentau_b200.policies.factory import make_policy, make_policy_config
from opentau_b200.policies.pi07.common import global_or_branch_decisions

FEATS = {"camera0": PolicyFeature(FeatureType.VISUAL, (3, 224, 224)), "state": PolicyFeature(FeatureType.STATE, (32,))}
OUT = {"actions": PolicyFeature(FeatureType.ACTION, (32,))}
G3 = dict(vlm=dict(TINY["vlm"], num_key_value_heads=2, sliding_window_pattern=2), vision=TINY["vision"],
          vlm_config={"tokens_per_image_side": 8})


def _ll(**kw):
    return make_policy(make_policy_config(
        "pi07_low_level", n_obs_steps=3, chunk_size=10, n_action_steps=10, prompt_max_length=16,
        discrete_action_max_length=8, discrete_action_vocab_size=256, dropout=0.0, device="cpu",
        resize_imgs_with_padding=(224, 224), metadata_max_length=12, response_max_length=8,
        spacetime_layer_stride=2, input_features=dict(FEATS), output_features=dict(OUT),
        expert=dict(TINY["expert"], num_key_value_heads=2), **G3, **kw), per_dataset_stats=[identity_stats()])


def _history_batch():
    b = tiny_batch()
    b["camera0"] = b["camera0"][:, None].repeat(1, 3, 1, 1, 1) * torch.tensor([0.5, 0.8, 1.0]).view(1, 3, 1, 1, 1)
    b["state"] = b["state"][:, None].repeat(1, 3, 1)
    b["obs_history_is_pad"] = torch.tensor([[1, 0, 0], [0, 0, 0], [1, 1, 0], [0, 0, 0]], dtype=torch.bool)
    return b


def test_temporal_pe_current_row_is_zero_and_alias_guard():
    pe = build_temporal_sinusoidal_pe(6, 32)
    assert pe.shape == (6, 32) and torch.all(pe[-1] == 0) and pe[0].abs().sum() > 0
    with pytest.raises(ValueError):
        build_temporal_sinusoidal_pe(50, 32, max_period=40.0)


def test_video_encoder_single_frame_equals_plain_siglip_and_history_matters():
    torch.manual_seed(0)
    pol = _ll()
    enc, vt = pol.model.video_encoder, pol.model.wrapper.gemma3.model.vision_tower
    x = torch.rand(2, 3, 224, 224) * 2 - 1
    assert torch.equal(enc(x[:, None]), vt(x))
    vid = torch.rand(2, 3, 3, 224, 224) * 2 - 1
    a = enc(vid)
    vid2 = vid.clone()
    vid2[:, 0] = torch.rand_like(vid2[:, 0])
    assert not torch.allclose(a, enc(vid2))                       # history reaches the current-frame tokens
    valid = torch.tensor([[False, True, True], [False, True, True]])
    assert torch.allclose(enc(vid, valid), enc(vid2, valid), atol=1e-5)   # ... unless that frame is padding
    # a forced history drop flags EVERY step as padding: the current frame is kept all the same, the result equals
    # "only the current frame is real" and is finite, and the caller's mask is not modified
    none_valid = torch.zeros(2, 3, dtype=torch.bool)
    only_current = torch.tensor([[False, False, True]] * 2)
    dropped = enc(vid, none_valid)
    assert torch.isfinite(dropped).all() and torch.allclose(dropped, enc(vid, only_current), atol=1e-6)
    assert not none_valid.any()
    assert not any("video_encoder" in k for k in pol.state_dict())    # no duplicated vision weights


def test_low_level_optional_blocks_and_training():
    torch.manual_seed(0)
    pol = _ll()
    b = _history_batch()
    base = pol(b, noise=torch.zeros(4, 10, 32), time=torch.full((4,), 0.5))
    b["response"] = ["grasp the cup", "", "move left", "open"]
    b["speed"] = torch.tensor([1, 2, 3, 4])
    b["robot_type"] = ["so101"] * 4
    b["subgoal0"] = torch.rand(4, 3, 224, 224)
    b["subgoal0_is_pad"] = torch.tensor([0, 1, 0, 0], dtype=torch.bool)
    rich = pol(b, noise=torch.zeros(4, 10, 32), time=torch.full((4,), 0.5))
    assert not torch.allclose(base["CE"], rich["CE"])
    (rich["MSE"] + rich["CE"]).backward()
    assert pol.model.state_proj.weight.grad.abs().sum() > 0
    pol.eval()
    assert pol.sample_actions(b).shape == (4, 10, 32)


def test_high_level_planner_ce_and_decoding():
    torch.manual_seed(0)
    hl = make_policy(make_policy_config(
        "pi07_high_level", prompt_max_length=16, memory_max_length=6, response_max_length=5, device="cpu",
        dropout=0.0, resize_imgs_with_padding=(224, 224), input_features=dict(FEATS), **G3))
    b = tiny_batch()
    b["next_memory"] = ["cup grasped"] * 4
    b["response"] = ["lift the cup"] * 4
    out = hl(b)
    assert out["MSE"].item() == 0 and out["CE"].item() > 0
    out["CE"].backward()
    assert not any("expert_layer" in n for n, _ in hl.named_parameters())
    mem, sub = hl.plan(b)
    assert len(mem) == 4 and len(sub) == 4
    with pytest.raises(NotImplementedError):
        hl.select_action(b)


def test_branch_decisions_single_process():
    assert global_or_branch_decisions((True, False), (True, False), ("a", "b"), torch.device("cpu")) == (True, False)
    with pytest.raises(ValueError):
        global_or_branch_decisions((False,), (True,), ("a",), torch.device("cpu"))


def _branch_worker(rank, world, port, diverge, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        present = (True, rank == 0) if diverge else (True, True)
        anys = (rank == 1, False)
        try:
            ret[rank] = global_or_branch_decisions(present, anys, ("response", "metadata"), torch.device("cpu"))
        except RuntimeError as e:
            ret[rank] = f"raised: {e}"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("diverge", [False, True])
def test_branch_decisions_two_ranks(diverge):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_branch_worker, args=(2, free_port(), diverge, ret), nprocs=2, join=True)
    if diverge:
        assert all(str(ret[r]).startswith("raised") and "metadata" in str(ret[r]) for r in (0, 1))
    else:
        assert ret[0] == ret[1] == (True, False)      # rank 1's "some real entries" wins on both ranks


def test_paligemma_variants_share_the_pi07_logic():
    """The legacy PaliGemma controller / planner: same behaviour, ``paligemma_with_expert`` checkpoint keys."""
    torch.manual_seed(0)
    ll = make_policy(make_policy_config(
        "pi07_paligemma_low_level", n_obs_steps=3, chunk_size=10, n_action_steps=10, prompt_max_length=16,
        discrete_action_max_length=8, discrete_action_vocab_size=256, dropout=0.0, device="cpu",
        metadata_max_length=12, response_max_length=8, spacetime_layer_stride=2, input_features=dict(FEATS),
        output_features=dict(OUT), **TINY), per_dataset_stats=[identity_stats()])
    b = _history_batch()
    b["response"] = ["grasp the cup", "", "move left", "open"]
    out = ll(b)
    (out["MSE"] + out["CE"]).backward()
    keys = set(ll.state_dict())
    assert any(k.startswith("model.paligemma_with_expert.paligemma.") for k in keys)
    assert not any("gemma3" in k or "video_encoder" in k for k in keys)
    ll.eval()
    assert ll.sample_actions(b).shape == (4, 10, 32)
    renamed = {k.replace("paligemma_with_expert", "gemma3_with_expert"): v for k, v in ll.state_dict().items()}
    assert set(type(ll)._fix_state_dict_keys(renamed, ll.config)) == keys

    hl = make_policy(make_policy_config(
        "pi07_paligemma_high_level_planner", prompt_max_length=16, memory_max_length=6, response_max_length=5,
        device="cpu", dropout=0.0, input_features=dict(FEATS), vlm=TINY["vlm"], vision=TINY["vision"]))
    hb = tiny_batch()
    hb["next_memory"], hb["response"] = ["cup grasped"] * 4, ["lift the cup"] * 4
    o = hl(hb)
    o["CE"].backward()
    assert o["CE"].item() > 0 and not any("gemma_expert" in n for n, _ in hl.named_parameters())
    mem, sub = hl.plan(hb)
    assert len(mem) == 4 and len(sub) == 4


def test_outlier_records_travel_from_forward_to_the_trainer(caplog):
    import logging

    from opentau_b200.parallel.engine import OptimHyper, TrainEngine
    from opentau_b200.scripts.train import update_policy
    torch.manual_seed(0)
    pol = _ll(warn_outlier_threshold=5.0)
    b = _history_batch()
    b["state"] = b["state"].clone()
    b["state"][2, -1, 3] = 80.0                                   # identity statistics: normalised value = raw value
    out = pol(b, noise=torch.zeros(4, 10, 32), time=torch.full((4,), 0.5))
    recs = out["outlier_records"]
    assert len(recs) == 1 and recs[0]["key"] == "state" and recs[0]["dim"] == 3 and abs(recs[0]["value"] - 80.0) < 1e-3
    clean = pol(_history_batch(), noise=torch.zeros(4, 10, 32), time=torch.full((4,), 0.5))
    assert clean["outlier_records"] == []
    engine = TrainEngine(pol, OptimHyper(lr=1e-4), device=torch.device("cpu"))
    with caplog.at_level(logging.WARNING):
        sums = update_policy(engine, [b])
    assert "outlier_records" not in sums and torch.isfinite(sums["loss"])
    assert any("normalised state dim 3" in r.getMessage() and "80.0" in r.getMessage() for r in caplog.records)


def test_keep_history_tokens_puts_every_frame_in_the_decoder():
    """Long-context variant: T frames x cameras stay in the decoder as frame blocks (reference drops them after the
    encoder); the prefix grows by (T - 1) x tokens-per-frame, padded history frames are masked, the model trains and
    samples, and the last frame block equals the default variant's only block."""
    torch.manual_seed(0)
    base, long = _ll(), _ll(keep_history_tokens=True)
    long.load_state_dict(base.state_dict())
    b = _history_batch()
    vid = b["camera0"] * 2 - 1
    e0 = base.model.embed_video(vid, None)
    e1 = long.model.embed_video(vid, None)
    assert e1.shape == (4, 3, *e0.shape[1:]) and torch.allclose(e1[:, -1], e0, atol=1e-5)
    lang = torch.randint(3, 1000, (4, 16))
    ones = torch.ones(4, 16, dtype=torch.bool)
    fv = b["obs_history_is_pad"]
    embs, pads, att, _ = long.model.embed_prefix([vid], [torch.ones(4, dtype=torch.bool)], lang, ones,
                                                  history_is_pad=fv)
    n = e0.shape[1]
    assert embs.shape[1] == 3 * n + 16
    assert not pads[0, :n].any() and pads[0, n:3 * n].all() and not pads[2, :2 * n].any() and pads[2, 2 * n:3 * n].all()
    blocks = torch.cumsum(att[0].int(), 0)
    assert blocks[0] == blocks[n - 1] and blocks[n] == blocks[0] + 1 and blocks[2 * n] == blocks[0] + 2
    long.train()
    out = long(b)
    (out["MSE"] + out["CE"]).backward()
    assert torch.isfinite(out["MSE"]) and torch.isfinite(out["CE"])
    long.eval()
    with torch.no_grad():
        a = long.sample_actions({k: v for k, v in b.items() if k != "actions"})
    assert a.shape[-2:] == (10, 32) and torch.isfinite(a).all()


def test_metadata_segment_text_is_reproduced_token_for_token():
    """The prefix's metadata segment is a fixed spelling: fields in one order, ``"<Label>: <value>, "`` joined by a space,
    behind ``"Metadata: "``; padded or absent fields are left out, a sample with none gets a masked empty segment."""
    pol = _ll()
    pol.config.metadata_max_length = 48
    seen = []
    real = pol.language_tokenizer

    class Spy:
        def __call__(self, texts, **kw):
            seen.append(list(texts))
            return real(texts, **kw)

        def __getattr__(self, name):
            return getattr(real, name)
    pol.language_tokenizer = Spy()
    state = torch.zeros(3, 32)
    batch = {"state": state, "speed": torch.tensor([30, 50, 70]), "speed_is_pad": torch.tensor([False, True, True]),
             "quality": torch.tensor([4, 4, 4]), "quality_is_pad": torch.tensor([False, False, True]),
             "mistake": torch.tensor([False, True, False]), "mistake_is_pad": torch.tensor([False, True, True]),
             "robot_type": ["so101", "", ""], "control_mode": ["ee", "joint", ""],
             "fps": torch.tensor([20, 20, 20]), "fps_is_pad": torch.tensor([False, False, True])}
    tokens, masks = pol.prepare_metadata(batch)
    assert seen[-1] == ["Metadata: Speed: 30,  Quality: 4,  Mistake: False,  Robot: so101,  FPS: 20,  Control: ee, ",
                        "Metadata: Quality: 4,  FPS: 20,  Control: joint, ", ""]
    assert tokens.shape == (3, 48) and masks[0].any() and masks[1].any() and not masks[2].any()
    assert pol.prepare_metadata({"state": state}) == (None, None)
    # what the evaluator injects from env.metadata goes through unchanged
    from opentau_b200.envs.configs import FakeEnvConfig, EnvMetadataConfig
    from opentau_b200.envs.utils import add_eval_metadata
    obs = add_eval_metadata({"state": state}, FakeEnvConfig(fps=15, metadata=EnvMetadataConfig(
        quality=5, mistake=False, control_mode="joint", emit_fps=True)))
    pol.prepare_metadata(obs)
    assert seen[-1] == ["Metadata: Quality: 5,  Mistake: False,  FPS: 15,  Control: joint, "] * 3


class _SpyTok:
    """Records the strings a policy hands to its tokenizer."""

    def __init__(self, real):
        self.real, self.seen = real, []

    def __call__(self, texts, **kw):
        self.seen.append(list(texts))
        return self.real(texts, **kw)

    def __getattr__(self, name):
        return getattr(self.real, name)


def test_prompt_spellings_follow_the_reference_checkpoints():
    """A checkpoint only understands the text layout it was trained on: every family's prompt / response strings are
    pinned here (separators spelled ``<eos>`` map to the separator id)."""
    import test_pi05_mem_cpu as mem
    import test_policies_cpu as fam
    from helpers import tiny_pi05
    b = {"state": torch.zeros(2, 32), "prompt": ["pick", "place"], "response": ["reach", ""]}
    pol = tiny_pi05(state_type="continuous")
    pol.language_tokenizer = spy = _SpyTok(pol.language_tokenizer)
    pol.prepare_language(b)
    assert spy.seen[-1] == ["Task: pick, ", "Task: place, "]
    pol = tiny_pi05()
    pol.language_tokenizer = spy = _SpyTok(pol.language_tokenizer)
    pol.prepare_language(b)
    assert spy.seen[-1][0].startswith("Task: pick, State: 128 128") and spy.seen[-1][0].endswith(";\n")
    pol = make_policy(mem._cfg(), per_dataset_stats=[identity_stats()])
    pol.language_tokenizer = spy = _SpyTok(pol.language_tokenizer)
    pol.prepare_language(b)
    assert spy.seen[-1] == ["Task: pick<eos>Actions:", "Task: place<eos>Actions:"]
    assert pol.language_tokenizer.real.encode("a<eos>b", add_special_tokens=False)[1] == pol.language_tokenizer.real.eos_token_id
    pol = make_policy(fam._pi06(), per_dataset_stats=[identity_stats()])
    pol.language_tokenizer = spy = _SpyTok(pol.language_tokenizer)
    pol.prepare_language(b)
    assert spy.seen[-1][1].startswith("Task: place<eos>State: 128") and spy.seen[-1][1].endswith("<eos>Actions:")
    pol.config.predict_response = True
    pol.prepare_language(b)
    assert spy.seen[-1][0].endswith("<eos>Response:")
    pol.prepare_response(b)
    assert spy.seen[-1] == ["reach<eos>Actions:", "<eos>Actions:"]
    ll = _ll()
    ll.language_tokenizer = spy = _SpyTok(ll.language_tokenizer)
    ll.prepare_language(b)
    assert spy.seen[-1] == ["Task: pick, ", "Task: place, "]
    _, masks = ll.prepare_response(b)
    assert spy.seen[-1] == ["Subtask: reach, ", ""] and masks[0].any() and not masks[1].any()
    hl = make_policy(make_policy_config(
        "pi07_high_level", prompt_max_length=48, memory_max_length=8, response_max_length=8, dropout=0.0, device="cpu",
        resize_imgs_with_padding=(224, 224), input_features=dict(FEATS), output_features=dict(OUT), **G3),
        per_dataset_stats=[identity_stats()])
    hl.language_tokenizer = spy = _SpyTok(hl.language_tokenizer)
    hl._lang({**b, "past_memory": ["opened the drawer", ""]}, torch.device("cpu"))
    assert spy.seen[-1][0].startswith("Task: pick, Past Memory: opened the drawer, State: 12")
    assert spy.seen[-1][0].endswith(", ")
