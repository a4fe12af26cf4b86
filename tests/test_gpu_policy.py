"""Every policy family on the GPU with a tiny geometry: forward, backward and sampling run through the native kernels
(shapes such as 72-wide vision heads, sliding windows, MRoPE and per-layer KV caches reach launchers that the pi0.5
tests never touch), and the loss agrees with the fp32 CPU statement of the same weights."""

import copy

import pytest
import torch

import test_pi05_mem_cpu as mem_cpu
import test_pi07_cpu as pi07_cpu
import test_policies_cpu as fam_cpu
import test_value_cpu as value_cpu
from helpers import tiny_batch
from opentau_b200.datasets.synthetic import identity_stats
from opentau_b200.policies.factory import make_policy

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _to_dev(b):
    return {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in b.items()}


def _run(pol_cpu, batch, sample_shape, atol=0.08, min_checked=5):
    """Same weights, same batch, same flow-matching noise and time on the CPU in fp32 and on the GPU in bf16 through
    the native kernels: both losses agree, and so do the gradients of every sizeable parameter (cosine)."""
    import inspect
    pol_cpu.train()
    for n, p in pol_cpu.named_parameters():        # open the zero-initialised adaptive-norm gates: the expert matters
        if ".dense." in n and p.requires_grad:
            torch.nn.init.normal_(p, std=0.05)
    pol = copy.deepcopy(pol_cpu).to(DEV).to(torch.bfloat16)
    kw_cpu, kw_gpu = {}, {}
    if "noise" in inspect.signature(pol_cpu.forward).parameters:
        cfg = pol_cpu.config
        B = next(v.shape[0] for v in batch.values() if isinstance(v, torch.Tensor))
        g = torch.Generator().manual_seed(11)
        noise = torch.randn(B, cfg.chunk_size, cfg.max_action_dim, generator=g)
        time = torch.rand(B, generator=g) * 0.8 + 0.1
        kw_cpu, kw_gpu = dict(noise=noise, time=time), dict(noise=noise.to(DEV), time=time.to(DEV))
    torch.manual_seed(5)
    want = pol_cpu(batch, **kw_cpu)
    torch.manual_seed(5)
    got = pol(_to_dev(batch), **kw_gpu)
    for k in ("MSE", "CE"):
        assert torch.isfinite(got[k]).all(), k
        if kw_cpu or k == "CE":                    # without injected noise the flow loss differs by its random draw
            assert abs(float(got[k]) - float(want[k])) <= atol * max(1.0, abs(float(want[k]))), k
    (got["MSE"] + got["CE"]).backward()
    (want["MSE"] + want["CE"]).backward()
    checked, worst = 0, (1.0, "")
    for (n, pc), (_, pg) in zip(pol_cpu.named_parameters(), pol.named_parameters()):
        if pc.grad is None or pg.grad is None or pc.numel() < 512 or float(pc.grad.abs().max()) < 1e-6:
            continue
        assert torch.isfinite(pg.grad).all(), n
        if not kw_cpu:
            continue
        cos = float(torch.nn.functional.cosine_similarity(pg.grad.float().cpu().flatten(), pc.grad.flatten(), dim=0))
        worst = min(worst, (cos, n))
        checked += 1
    if kw_cpu:
        assert checked >= min_checked and worst[0] > 0.95, (checked, worst)
    if sample_shape is not None:
        pol.eval()
        a = pol.sample_actions(_to_dev(batch))
        assert tuple(a.shape) == sample_shape and torch.isfinite(a).all()
    from opentau_b200.ops import cuda_ops
    cuda_ops.check_status()


@pytest.mark.parametrize("builder", [fam_cpu._pi06, fam_cpu._pi0, fam_cpu._cosmos3])
def test_family_forward_backward_sample(builder):
    torch.manual_seed(0)
    _run(make_policy(builder(), per_dataset_stats=[identity_stats()]), tiny_batch(), (4, 10, 32))


@pytest.mark.parametrize("use_motion", [False, True])
def test_pi05_mem(use_motion):
    torch.manual_seed(0)
    pol = make_policy(mem_cpu._cfg(use_motion=use_motion), per_dataset_stats=[identity_stats()])
    _run(pol, mem_cpu._hist_batch(), (2, 10, 32))


def test_pi07_low_level():
    torch.manual_seed(0)
    _run(pi07_cpu._ll(), pi07_cpu._history_batch(), (4, 10, 32))


def test_value_model():
    torch.manual_seed(0)
    pol = make_policy(value_cpu._cfg(), per_dataset_stats=[identity_stats()])
    _run(pol, value_cpu._batch(), None)


def test_cosmos3_cuda_graph_sampler_matches_eager():
    from opentau_b200.scripts.benchmark_inference import build_cosmos3
    policy, batch = build_cosmos3(2, 16, torch.device(DEV), tiny=True, num_steps=3)
    noise = torch.randn(1, 50, 32, device=DEV)
    want = policy.sample_actions(batch, noise=noise)
    policy.enable_cuda_graphs(True)
    got = policy.sample_actions(batch, noise=noise)
    again = policy.sample_actions(batch, noise=noise)
    torch.testing.assert_close(got, want, atol=1e-3, rtol=1e-3)
    assert torch.equal(got, again)


def test_spacetime_video_encoder_matches_cpu():
    """The SpaceTime SigLIP encoder (temporal-causal attention through the block-causal kernel, then spatial
    attention) on the GPU in bf16 against its CPU fp32 statement, with a padded history frame."""
    torch.manual_seed(0)
    pol = pi07_cpu._ll()
    enc = pol.model.video_encoder
    vid = torch.rand(2, 3, 3, 224, 224) * 2 - 1
    valid = torch.tensor([[False, True, True], [True, True, True]])
    with torch.no_grad():
        want = enc(vid, valid)
        want_all = enc(vid, valid, keep_history=True)
    gpu = copy.deepcopy(pol).to(DEV).to(torch.bfloat16)
    genc = gpu.model.video_encoder
    with torch.no_grad():
        got = genc(vid.to(DEV).to(torch.bfloat16), valid.to(DEV))
        got_all = genc(vid.to(DEV).to(torch.bfloat16), valid.to(DEV), keep_history=True)
    torch.testing.assert_close(got.float().cpu(), want, rtol=6e-2, atol=6e-2)
    assert got_all.shape == want_all.shape == (2, 3, *want.shape[1:])
    torch.testing.assert_close(got_all[:, -1].float().cpu(), want_all[:, -1], rtol=6e-2, atol=6e-2)
    from opentau_b200.ops import cuda_ops
    cuda_ops.check_status()


def test_loss_curves_of_native_and_oracle_paths_agree(monkeypatch):
    """50 optimizer steps of the tiny pi0.5 through the hand-written kernels and through the plain-PyTorch
    statement of the same model (same weights, batch, noise, time, fp32 masters): the two loss curves stay together
    to bf16 tolerance and both go down."""
    from helpers import tiny_pi05
    from opentau_b200.ops import cuda_ops
    from opentau_b200.parallel.engine import OptimHyper, TrainEngine
    b = tiny_batch(device=DEV)
    g = torch.Generator().manual_seed(3)
    noise, time = torch.randn(4, 10, 32, generator=g).to(DEV), (torch.rand(4, generator=g) * 0.8 + 0.1).to(DEV)
    curves = {}
    for mode in ("native", "oracle"):
        if mode == "oracle":
            monkeypatch.setenv("OPENTAU_B200_ORACLE", "1")
        else:
            monkeypatch.delenv("OPENTAU_B200_ORACLE", raising=False)
        pol = tiny_pi05(seed=4).to(torch.bfloat16).train()
        eng = TrainEngine(pol, OptimHyper(lr=1e-3, grad_clip_norm=1.0), device=DEV)
        losses = []
        for _ in range(50):
            out = pol(b, noise=noise, time=time)
            loss = out["MSE"] + out["CE"]
            loss.backward()
            eng.optimizer_step()
            losses.append(float(loss))
        curves[mode] = losses
    monkeypatch.delenv("OPENTAU_B200_ORACLE", raising=False)
    cuda_ops.check_status()
    a, o = curves["native"], curves["oracle"]
    assert a[-1] < 0.8 * a[0] and o[-1] < 0.8 * o[0]
    rel = [abs(x - y) / max(abs(y), 1e-6) for x, y in zip(a, o)]
    # early steps agree to bf16 rounding; later, with the loss of this one batch driven towards zero, two bf16
    # trajectories drift apart in RELATIVE terms, so the whole curve is held to a tolerance in units of the initial loss
    scaled = [abs(x - y) / o[0] for x, y in zip(a, o)]
    assert max(rel[:10]) < 0.03 and max(scaled) < 0.03, (max(rel[:10]), max(scaled), max(rel))


def test_response_decoding_on_the_gpu_matches_the_teacher_forced_pass():
    """The token-by-token decode appends keys / values in place behind the prefix through the fused kernels; one full
    pass over the same text must predict the same tokens."""
    from helpers import tiny_pi05
    from opentau_b200 import ops
    pol = tiny_pi05(predict_response=True, response_max_length=6).to(DEV).to(torch.bfloat16).eval()
    model, cfg = pol.model, pol.config
    b = _to_dev(tiny_batch())
    B = b["state"].shape[0]
    actions = pol.sample_actions(b)
    toks, masks = model.last_response_tokens, model.last_response_masks
    assert toks.shape == (B, 6) and torch.isfinite(actions.float()).all() and len(pol.last_response) == B
    idx = pol._resolve_dataset_index(b, B, b["state"].device)
    nb = pol.normalize_inputs(b, idx)
    images, img_masks = pol.prepare_images(nb)
    lang_tokens, lang_masks = pol.prepare_language(nb)
    embs, pad, att, pos = model.embed_prefix(images, img_masks, lang_tokens, lang_masks, response_tokens=toks,
                                             response_masks=masks)
    blk, valid = ops.make_block_ids(pad, att)
    pos = torch.cumsum(pad, dim=1) - 1 if pos is None else pos
    with torch.no_grad():
        (out, _), _ = model.wrapper(inputs_embeds=[embs, None], position_ids=pos, q_blk=blk, q_valid=valid)
    logits = ops.linear(out[:, -6:], model.wrapper.lm_head_weight()).float()
    top2 = logits.topk(2, dim=-1)
    for i in range(5):
        live = masks[:, i + 1]
        same = top2.indices[:, i, 0] == toks[:, i + 1]
        # bf16: a near-tie between the two best logits may flip between the incremental and the full pass
        near_tie = (top2.values[:, i, 0] - top2.values[:, i, 1]) < 0.05 * top2.values[:, i, 0].abs().clamp(min=1.0)
        assert bool((same | near_tie | ~live).all()), i
