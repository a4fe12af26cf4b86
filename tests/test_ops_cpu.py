"""Hand-written autograd functions (ops.fused) against plain autograd of the reference bodies, fp32 CPU."""

import math

import pytest
import torch

from opentau_b200 import ops
from opentau_b200.ops import fused, prims, reference as ref


def _grads(fn, inputs):
    out = fn(*inputs)
    outs = out if isinstance(out, tuple) else (out,)
    loss = sum((o.float() * torch.linspace(0.5, 1.5, o.numel()).view_as(o)).sum() for o in outs if o is not None)
    return out, torch.autograd.grad(loss, [i for i in inputs if i.requires_grad], allow_unused=True)


def _leaf(*shape, scale=1.0):
    return (torch.randn(*shape, dtype=torch.float64) * scale).float().requires_grad_()


def test_linear_matches_reference():
    torch.manual_seed(0)
    x, w, b, r = _leaf(3, 5, 16), _leaf(24, 16), _leaf(24), _leaf(3, 5, 24)
    o1, g1 = _grads(lambda *a: fused.linear(*a), (x, w, b, r))
    o2, g2 = _grads(lambda *a: ref.linear(*a), (x, w, b, r))
    torch.testing.assert_close(o1, o2)
    for a, c in zip(g1, g2):
        torch.testing.assert_close(a, c, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("unit_offset", [True, False])
def test_rms_norm(unit_offset):
    torch.manual_seed(1)
    x, w = _leaf(4, 7, 32), _leaf(32, scale=0.1)
    o1, g1 = _grads(lambda a, b: fused.rms_norm(a, b, 1e-6, unit_offset), (x, w))
    o2, g2 = _grads(lambda a, b: ref.rms_norm(a, b, 1e-6, unit_offset), (x, w))
    torch.testing.assert_close(o1, o2)
    for a, c in zip(g1, g2):
        torch.testing.assert_close(a, c, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("per_token", [True, False])
def test_ada_rms_norm(per_token):
    torch.manual_seed(2)
    x = _leaf(3, 6, 16)
    mod = _leaf(3, 6, 48, scale=0.3) if per_token else _leaf(3, 48, scale=0.3)
    o1, g1 = _grads(lambda a, m: fused.ada_rms_norm(a, m, 1e-6), (x, mod))
    o2, g2 = _grads(lambda a, m: ref.ada_rms_norm(a, m, 1e-6), (x, mod))
    torch.testing.assert_close(o1[0], o2[0])
    torch.testing.assert_close(o1[1].expand_as(o2[1]), o2[1])
    for a, c in zip(g1, g2):
        torch.testing.assert_close(a, c, rtol=1e-4, atol=1e-5)


def test_layer_norm():
    torch.manual_seed(3)
    x, w, b = _leaf(5, 24), _leaf(24), _leaf(24)
    o1, g1 = _grads(lambda *a: fused.layer_norm(*a, 1e-6), (x, w, b))
    o2, g2 = _grads(lambda *a: ref.layer_norm(*a, 1e-6), (x, w, b))
    torch.testing.assert_close(o1, o2, rtol=1e-5, atol=1e-5)
    for a, c in zip(g1, g2):
        torch.testing.assert_close(a, c, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
def test_gated_mlp(act):
    torch.manual_seed(4)
    x, wg, wu, wd, r = _leaf(2, 5, 16), _leaf(64, 16, scale=0.3), _leaf(64, 16, scale=0.3), _leaf(16, 64, scale=0.3), _leaf(2, 5, 16)
    w_gu = prims.interleave_gate_up(wg.detach(), wu.detach()).requires_grad_()

    def plain(x, wg, wu, wd, r):
        h = ref.act_fn(x @ wg.t(), act) * (x @ wu.t())
        return h @ wd.t() + r

    o1, g1 = _grads(lambda x, w, d, r: fused.gated_mlp(x, w, d, act, r), (x, w_gu, wd, r))
    o2, g2 = _grads(plain, (x, wg, wu, wd, r))
    torch.testing.assert_close(o1, o2, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(g1[0], g2[0], rtol=1e-4, atol=1e-5)
    dg, du = prims.deinterleave_gate_up(g1[1])
    torch.testing.assert_close(dg, g2[1], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(du, g2[2], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(g1[2], g2[3], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(g1[3], g2[4])


def test_interleave_roundtrip():
    g, u = torch.randn(64, 8), torch.randn(64, 8)
    g2, u2 = prims.deinterleave_gate_up(prims.interleave_gate_up(g, u))
    assert torch.equal(g, g2) and torch.equal(u, u2)


def test_rope_inverse_is_backward():
    torch.manual_seed(5)
    x = _leaf(2, 6, 3, 16)
    pos = torch.arange(6)[None].expand(2, -1)
    cos, sin = ops.rope_angles(pos, 16, 10000.0)
    o1, g1 = _grads(lambda a: fused.rope(a, cos, sin), (x,))
    o2, g2 = _grads(lambda a: ref.apply_rope(a, cos, sin), (x,))
    torch.testing.assert_close(o1, o2)
    torch.testing.assert_close(g1[0], g2[0], rtol=1e-5, atol=1e-6)


def _mask_case(B, Sq, Sk, cross=0):
    att = torch.zeros(B, Sq, dtype=torch.bool)
    att[:, Sq // 2:] = True   # second half causal
    pad = torch.ones(B, Sq, dtype=torch.bool)
    pad[0, -1] = False
    q_blk, q_valid = ops.make_block_ids(pad, att)
    if cross:
        k_blk = torch.cat([torch.full((B, cross), ops.INT_MIN, dtype=torch.int32), q_blk], 1)
        k_valid = torch.cat([torch.ones(B, cross, dtype=torch.bool), q_valid], 1)
        k_valid[1, 0] = False
    else:
        k_blk, k_valid = q_blk, q_valid
    return q_blk, k_blk, q_valid, k_valid


@pytest.mark.parametrize("cross", [0, 5])
@pytest.mark.parametrize("hkv", [1, 2])
def test_block_attention(cross, hkv):
    torch.manual_seed(6)
    B, Sq, H, D = 2, 8, 4, 16
    Sk = Sq + cross
    q, k, v = _leaf(B, Sq, H, D), _leaf(B, Sk, hkv, D), _leaf(B, Sk, hkv, D)
    qb, kb, qv, kv = _mask_case(B, Sq, Sk, cross)
    scale = D ** -0.5
    o1, g1 = _grads(lambda *a: fused.block_attention(*a, qb, kb, qv, kv, scale), (q, k, v))
    o2, g2 = _grads(lambda *a: ref.block_attention(*a, qb, kb, qv, kv, scale), (q, k, v))
    valid = qv[:, :, None].expand(B, Sq, H * D)
    torch.testing.assert_close(o1[valid], o2[valid], rtol=1e-4, atol=1e-5)
    # gradients: padded query rows contribute differently (uniform softmax vs zeros) only through
    # rows that are invalid, which carry no weight in the reference either when masked out
    o1b, g1b = _grads(lambda *a: fused.block_attention(*a, qb, kb, qv, kv, scale) * valid, (q, k, v))
    o2b, g2b = _grads(lambda *a: ref.block_attention(*a, qb, kb, qv, kv, scale) * valid, (q, k, v))
    for a, c in zip(g1b, g2b):
        torch.testing.assert_close(a, c, rtol=1e-4, atol=1e-5)


def test_block_ids_reproduce_dense_mask():
    from opentau_b200.policies.pi05.modeling_pi05 import make_att_2d_masks
    pad = torch.tensor([[1, 1, 1, 1, 0, 1], [1, 1, 0, 1, 1, 1]], dtype=torch.bool)
    for att_row in ([1, 1, 1, 1, 1, 1], [0, 0, 0, 1, 1, 1], [1, 0, 1, 0, 1, 0], [0, 0, 0, 0, 0, 0]):
        att = torch.tensor([att_row, att_row])
        cs = torch.cumsum(att, 1)
        expect = (cs[:, None, :] <= cs[:, :, None]) & (pad[:, None, :] & pad[:, :, None])
        assert torch.equal(make_att_2d_masks(pad, att), expect)
    cross_pad = torch.tensor([[1, 0, 1], [1, 1, 1]], dtype=torch.bool)
    m = make_att_2d_masks(pad, att, n_cross_att_tokens=3, cross_att_pad_masks=cross_pad)
    assert m.shape == (2, 6, 9)
    assert torch.equal(m[:, :, :3], pad[:, :, None] & cross_pad[:, None, :])


def test_linear_cross_entropy():
    torch.manual_seed(7)
    h, w, b = _leaf(10, 16), _leaf(32, 16), _leaf(32)
    labels = torch.randint(0, 32, (10,))
    o1, g1 = _grads(lambda *a: fused.linear_cross_entropy(*a, labels), (h, w, b))
    o2, g2 = _grads(lambda *a: ref.linear_cross_entropy(*a, labels), (h, w, b))
    torch.testing.assert_close(o1, o2, rtol=1e-5, atol=1e-5)
    for a, c in zip(g1, g2):
        torch.testing.assert_close(a, c, rtol=1e-4, atol=1e-5)


def test_masked_mse_contract():
    u = torch.randn(2, 4, 6)
    v = torch.randn(2, 4, 6)
    pad = torch.tensor([[0, 0, 0, 1], [0, 0, 0, 0]], dtype=torch.bool)
    rad = torch.tensor([3, 6])
    loss = ops.flow_matching_masked_mse(u, v, None, pad, rad)
    mask = torch.ones(2, 4, 6, dtype=torch.bool)
    mask[0, 3] = False
    mask[0, :, 3:] = False
    expect = ((u - v) ** 2 * mask).sum() / (mask.sum() + 1e-8)
    torch.testing.assert_close(loss, expect)


def test_time_embedding_and_beta_time():
    t = torch.tensor([[0.0, 0.5, 1.0]])
    e = ops.sinusoidal_time_embedding(t, 8)
    assert e.shape == (1, 3, 8)
    frac = torch.linspace(0, 1, 4, dtype=torch.float64)
    period = 4e-3 * (4.0 / 4e-3) ** frac
    torch.testing.assert_close(e[0, 1, :4], torch.sin(2 * math.pi / period * 0.5).float())
    from opentau_b200.policies.pi05.modeling_pi05 import PI05FlowMatching
    torch.manual_seed(0)
    s = PI05FlowMatching.sample_time(20000, "cpu")
    assert 0.001 <= s.min() and s.max() <= 1.0
    assert abs(s.mean().item() - (0.6 * 0.999 + 0.001)) < 0.01   # Beta(1.5,1) has mean 0.6


def test_adamw_flat_matches_torch():
    torch.manual_seed(8)
    p = torch.randn(100)
    ref_p = p.clone().requires_grad_()
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v, p32 = torch.zeros(100), torch.zeros(100), p.clone()
    for step in range(1, 4):
        g = torch.randn(100)
        ref_p.grad = g.clone()
        opt.step()
        ref.adamw_flat(p32, g, m, v, None, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
        torch.testing.assert_close(p32, ref_p.detach(), rtol=1e-5, atol=1e-6)


def test_resize_with_pad_semantics():
    img = torch.rand(1, 3, 100, 200)
    out = ops.resize_with_pad(img, 224, 224, pad_value=0.0)
    assert out.shape == (1, 3, 224, 224)
    assert torch.all(out[:, :, :112, :] == 0)      # padding is on the top
    assert out[:, :, 112:, :].abs().sum() > 0


def test_forked_norms_give_the_gradients_of_norm_plus_residual():
    """``rms_norm_fork`` / ``ada_rms_norm_fork``: same values as the plain norms, and the gradient of x through
    (branch on the norm) + (residual on the second output) equals the plain two-path graph, including when only one of
    the two outputs is used."""
    import torch

    from opentau_b200 import ops
    torch.manual_seed(0)
    x = torch.randn(2, 5, 16, requires_grad=True)
    w = torch.randn(16, requires_grad=True)
    mod = torch.randn(2, 48, requires_grad=True)
    lin = torch.randn(16, 16)

    def plain():
        h = ops.rms_norm(x, w, 1e-6, True)
        y = x + h @ lin
        h2, gate = ops.ada_rms_norm(y, mod, 1e-6)
        return (y + gate * (h2 @ lin)).square().sum()

    def forked():
        h, xr = ops.rms_norm_fork(x, w, 1e-6, True)
        y = xr + h @ lin
        h2, gate, yr = ops.ada_rms_norm_fork(y, mod, 1e-6)
        return (yr + gate * (h2 @ lin)).square().sum()

    ga = torch.autograd.grad(plain(), (x, w, mod))
    gb = torch.autograd.grad(forked(), (x, w, mod))
    for a, b in zip(ga, gb):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-5)
    assert torch.allclose(plain(), forked())
    h, xr = ops.rms_norm_fork(x, w)
    torch.testing.assert_close(torch.autograd.grad(xr.sum(), x)[0], torch.ones_like(x))      # residual path alone
    h, xr = ops.rms_norm_fork(x, w)
    torch.testing.assert_close(torch.autograd.grad(h.sum(), x)[0], torch.autograd.grad(ops.rms_norm(x, w).sum(), x)[0])
    with torch.no_grad():
        h, xr = ops.rms_norm_fork(x, w)
        assert xr is x                                                                       # nothing to fork
