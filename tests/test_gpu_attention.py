"""tcgen05 block-causal attention against the dense fp32 reference (run on a B200)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(B, Sq, H, Hkv, D, cross, dev, seed=0, pad=True, causal_from=None):
    g = torch.Generator().manual_seed(seed)
    Sk = Sq + cross
    q = (torch.randn(B, Sq, H, D, generator=g)).to(torch.bfloat16).to(dev)
    k = (torch.randn(B, Sk, Hkv, D, generator=g)).to(torch.bfloat16).to(dev)
    v = (torch.randn(B, Sk, Hkv, D, generator=g)).to(torch.bfloat16).to(dev)
    att = torch.zeros(B, Sq, dtype=torch.bool)
    cf = Sq // 2 if causal_from is None else causal_from
    att[:, cf:] = True
    padm = torch.ones(B, Sq, dtype=torch.bool)
    if pad:
        padm[0, -3:] = False
        if Sq > 20:
            padm[-1, 5:9] = False
    from opentau_b200 import ops
    q_blk, q_valid = ops.make_block_ids(padm, att)
    if cross:
        k_blk = torch.cat([torch.full((B, cross), ops.INT_MIN, dtype=torch.int32), q_blk], 1)
        cv = torch.ones(B, cross, dtype=torch.bool)
        if pad:
            cv[0, 1::7] = False
        k_valid = torch.cat([cv, q_valid], 1)
    else:
        k_blk, k_valid = q_blk, q_valid
    return q, k, v, q_blk.to(dev), k_blk.to(dev), q_valid.to(dev), k_valid.to(dev)


@pytest.mark.parametrize("D", [64, 72, 128, 256])
@pytest.mark.parametrize("H,Hkv", [(8, 1), (8, 4), (4, 4), (16, 8)])
@pytest.mark.parametrize("Sq,cross", [(50, 0), (131, 0), (50, 203), (300, 0), (64, 64)])
def test_attn_fwd_matches_dense(D, H, Hkv, Sq, cross):
    from opentau_b200 import ops
    from opentau_b200.ops import attention_native, cuda_ops
    dev = torch.device("cuda:0")
    B = 2
    q, k, v, qb, kb, qv, kv = _case(B, Sq, H, Hkv, D, cross, dev, seed=D + Sq)
    scale = D ** -0.5
    assert attention_native.supported(q, k, v)
    o, lse = attention_native.attn_fwd(q, k, v, qb, kb, qv, kv, scale)
    cuda_ops.check_status()
    o_ref, lse_ref = ops.prims.attn_fwd(q.cpu().float(), k.cpu().float(), v.cpu().float(), qb.cpu(), kb.cpu(),
                                        qv.cpu(), kv.cpu(), scale)
    valid = qv.cpu()
    od = o.cpu().float().view(B, Sq, H, D)[valid]
    ord_ = o_ref.view(B, Sq, H, D)[valid]
    torch.testing.assert_close(od, ord_, rtol=3e-2, atol=3e-2)
    lv = lse.cpu().permute(0, 2, 1)[valid]
    lr = lse_ref.permute(0, 2, 1)[valid]
    torch.testing.assert_close(lv, lr, rtol=1e-2, atol=2e-2)
    assert torch.isfinite(o.float()).all()


def test_attn_fwd_strided_qkv_views():
    """q/k/v as column slices of one fused projection output (the layout the model produces)."""
    from opentau_b200 import ops
    from opentau_b200.ops import attention_native, cuda_ops
    dev = torch.device("cuda:0")
    B, S, H, Hkv, D = 2, 200, 8, 1, 256
    qkv = torch.randn(B, S, (H + 2 * Hkv) * D, device=dev).to(torch.bfloat16)
    q, k, v = qkv.split([H * D, Hkv * D, Hkv * D], dim=-1)
    q, k, v = q.unflatten(-1, (H, D)), k.unflatten(-1, (Hkv, D)), v.unflatten(-1, (Hkv, D))
    blk = torch.zeros(B, S, dtype=torch.int32, device=dev)
    ok = torch.ones(B, S, dtype=torch.bool, device=dev)
    o, _ = attention_native.attn_fwd(q, k, v, blk, blk, ok, ok, D ** -0.5)
    cuda_ops.check_status()
    o_ref = ops.ref.block_attention(q.float().cpu(), k.float().cpu(), v.float().cpu(), blk.cpu(), blk.cpu(),
                                    ok.cpu(), ok.cpu(), D ** -0.5)
    torch.testing.assert_close(o.cpu().float(), o_ref, rtol=3e-2, atol=3e-2)


def test_attn_large_logits_trigger_rescale():
    """Row maxima that grow late in the key sequence exercise the lazy O-rescale path."""
    from opentau_b200 import ops
    from opentau_b200.ops import attention_native, cuda_ops
    dev = torch.device("cuda:0")
    B, S, H, D = 1, 512, 4, 64
    q = torch.randn(B, S, H, D, device=dev).to(torch.bfloat16)
    k = torch.randn(B, S, H, D, device=dev).to(torch.bfloat16)
    k[:, 400:] *= 6.0
    v = torch.randn(B, S, H, D, device=dev).to(torch.bfloat16)
    blk = torch.zeros(B, S, dtype=torch.int32, device=dev)
    ok = torch.ones(B, S, dtype=torch.bool, device=dev)
    o, lse = attention_native.attn_fwd(q, k, v, blk, blk, ok, ok, 1.0)
    cuda_ops.check_status()
    o_ref, lse_ref = ops.prims.attn_fwd(q.cpu().float(), k.cpu().float(), v.cpu().float(), blk.cpu(), blk.cpu(),
                                        ok.cpu(), ok.cpu(), 1.0)
    torch.testing.assert_close(o.cpu().float(), o_ref, rtol=5e-2, atol=5e-2)
    torch.testing.assert_close(lse.cpu(), lse_ref, rtol=1e-2, atol=5e-2)


def test_attention_autograd_on_gpu_matches_cpu():
    from opentau_b200 import ops
    dev = torch.device("cuda:0")
    B, Sq, H, Hkv, D = 2, 70, 8, 1, 64
    q, k, v, qb, kb, qv, kv = _case(B, Sq, H, Hkv, D, 30, dev, seed=3)
    qc, kc, vc = (t.cpu().float().requires_grad_() for t in (q, k, v))
    q, k, v = (t.requires_grad_() for t in (q, k, v))
    o = ops.block_attention(q, k, v, qb, kb, qv, kv, D ** -0.5)
    oc = ops.block_attention(qc, kc, vc, qb.cpu(), kb.cpu(), qv.cpu(), kv.cpu(), D ** -0.5)
    w = torch.randn_like(oc) * qv.cpu()[:, :, None]
    (o.float() * w.to(dev)).sum().backward()
    (oc * w).sum().backward()
    for a, c in ((q.grad, qc.grad), (k.grad, kc.grad), (v.grad, vc.grad)):
        torch.testing.assert_close(a.cpu().float(), c, rtol=5e-2, atol=5e-2)


@pytest.mark.parametrize("D", [64, 72, 128, 256])
@pytest.mark.parametrize("H,Hkv", [(8, 1), (8, 4), (4, 4)])
@pytest.mark.parametrize("Sq,cross", [(50, 0), (131, 0), (50, 203), (300, 0)])
def test_attn_bwd_matches_dense(D, H, Hkv, Sq, cross):
    from opentau_b200 import ops
    from opentau_b200.ops import attention_native, cuda_ops
    dev = torch.device("cuda:0")
    B = 2
    q, k, v, qb, kb, qv, kv = _case(B, Sq, H, Hkv, D, cross, dev, seed=7 * D + Sq)
    scale = D ** -0.5
    assert attention_native.supported_bwd(q, k, v)
    o, lse = attention_native.attn_fwd(q, k, v, qb, kb, qv, kv, scale)
    g = torch.Generator().manual_seed(5)
    do = (torch.randn(B, Sq, H * D, generator=g) * qv.cpu()[:, :, None]).to(torch.bfloat16).to(dev)
    dq, dk, dv = attention_native.attn_bwd(do, q, k, v, o, lse, qb, kb, qv, kv, scale)
    cuda_ops.check_status()
    qc, kc, vc = q.cpu().float(), k.cpu().float(), v.cpu().float()
    o_ref, lse_ref = ops.prims.attn_fwd(qc, kc, vc, qb.cpu(), kb.cpu(), qv.cpu(), kv.cpu(), scale)
    dqr, dkr, dvr = ops.prims.attn_bwd(do.cpu().float(), qc, kc, vc, o_ref, lse_ref, qb.cpu(), kb.cpu(), qv.cpu(),
                                        kv.cpu(), scale)
    valid_q = qv.cpu()
    torch.testing.assert_close(dq.cpu().float()[valid_q], dqr[valid_q], rtol=5e-2, atol=5e-2)
    valid_k = kv.cpu()
    torch.testing.assert_close(dk.cpu().float()[valid_k], dkr[valid_k], rtol=5e-2, atol=8e-2)
    torch.testing.assert_close(dv.cpu().float()[valid_k], dvr[valid_k], rtol=5e-2, atol=8e-2)
    assert torch.isfinite(dq.float()).all() and torch.isfinite(dk.float()).all() and torch.isfinite(dv.float()).all()


@pytest.mark.parametrize("B,Sq,Sk,H,Hkv,D", [(1, 51, 1019, 8, 1, 256), (2, 51, 700, 16, 8, 128), (1, 10, 300, 4, 4, 64),
                                             (1, 51, 1019, 8, 8, 72)])
@pytest.mark.parametrize("nsplit", [2, 5, 8])
def test_split_kv_matches_single_pass(B, Sq, Sk, H, Hkv, D, nsplit):
    """A suffix attending to a cached prefix plus itself: the key blocks split over several CTAs and merged give the
    single-pass result (also when some splits reach no visible key)."""
    from opentau_b200.ops import attention_native, cuda_ops
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    q = torch.randn(B, Sq, H, D, device=dev).to(torch.bfloat16)
    k = torch.randn(B, Sk, Hkv, D, device=dev).to(torch.bfloat16)
    v = torch.randn(B, Sk, Hkv, D, device=dev).to(torch.bfloat16)
    P = Sk - Sq
    k_blk = torch.cat([torch.full((B, P), -2**31, dtype=torch.int32, device=dev),
                       torch.arange(Sq, device=dev, dtype=torch.int32)[None].expand(B, -1) // 7], 1).contiguous()
    q_blk = k_blk[:, P:].contiguous()
    k_valid = torch.rand(B, Sk, device=dev) > 0.1
    q_valid = torch.ones(B, Sq, dtype=torch.bool, device=dev)
    q_valid[:, -3:] = False
    scale = D ** -0.5
    want_o, want_lse = attention_native.attn_fwd(q, k, v, q_blk, k_blk, q_valid, k_valid, scale, nsplit=1)
    got_o, got_lse = attention_native.attn_fwd(q, k, v, q_blk, k_blk, q_valid, k_valid, scale, nsplit=nsplit)
    cuda_ops.check_status()
    torch.testing.assert_close(got_o.float(), want_o.float(), atol=1e-2, rtol=1e-2)
    torch.testing.assert_close(got_lse, want_lse, atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("D", [32, 72, 128, 160, 256])
@pytest.mark.parametrize("H,Hkv", [(8, 1), (6, 3), (4, 4)])
@pytest.mark.parametrize("Sq,cross", [(50, 0), (131, 0), (50, 203), (33, 64)])
def test_fp32_attention_kernels_match_the_dense_fp32_reference(D, H, Hkv, Sq, cross, monkeypatch):
    """The exact fp32 kernels (forward, dQ, dK / dV over the whole GQA group) against the CPU fp32 dense evaluation,
    at fp32 tolerances: block-causal mask, pads, a cross-attention prefix with block id INT_MIN, strided inputs."""
    from opentau_b200 import ops
    from opentau_b200.ops import attention_native
    dev = torch.device("cuda:0")
    B = 2
    qh, kh, vh, qb, kb, qv, kv = _case(B, Sq, H, Hkv, D, cross, dev, seed=3 * D + Sq)
    g = torch.Generator().manual_seed(11)
    Sk = Sq + cross
    # q as a strided view of a fused (B, Sq, H + 2 Hkv, D) projection, as the models produce it
    fused = torch.randn(B, Sq, H + 2 * Hkv, D, generator=g).to(dev)
    q = fused[:, :, :H]
    k = torch.randn(B, Sk, Hkv, D, generator=g).to(dev)
    v = torch.randn(B, Sk, Hkv, D, generator=g).to(dev)
    scale = D ** -0.5
    assert attention_native.supported_f32(q, k, v) and not attention_native.supported(q, k, v)
    from opentau_b200.ops import attention as dispatch
    monkeypatch.setenv("OPENTAU_B200_F32_ATTN", "kernel")               # at small sizes "auto" may take the dense body
    o, lse = dispatch.attn_fwd(q, k, v, qb, kb, qv, kv, scale)
    assert attention_native.prefer_f32_kernels(q, k)
    monkeypatch.setenv("OPENTAU_B200_F32_ATTN", "auto")
    assert attention_native.prefer_f32_kernels(q, k) == (D <= 128)      # these score tensors are far below the limit
    qc, kc, vc = q.cpu().contiguous(), k.cpu(), v.cpu()
    o_ref, lse_ref = ops.prims.attn_fwd(qc, kc, vc, qb.cpu(), kb.cpu(), qv.cpu(), kv.cpu(), scale)
    vq, vk = qv.cpu(), kv.cpu()
    torch.testing.assert_close(o.cpu().view(B, Sq, H, D)[vq], o_ref.view(B, Sq, H, D)[vq], rtol=2e-4, atol=2e-5)
    torch.testing.assert_close(lse.cpu().permute(0, 2, 1)[vq], lse_ref.permute(0, 2, 1)[vq], rtol=1e-5, atol=2e-5)
    do = (torch.randn(B, Sq, H * D, generator=g) * vq[:, :, None]).to(dev)
    dq, dk, dv = attention_native.attn_f32_bwd(do, q, k, v, o, lse, qb, kb, qv, kv, scale)
    dqr, dkr, dvr = ops.prims.attn_bwd(do.cpu(), qc, kc, vc, o_ref, lse_ref, qb.cpu(), kb.cpu(), vq, vk, scale)
    torch.testing.assert_close(dq.cpu()[vq], dqr[vq], rtol=5e-4, atol=5e-5)
    torch.testing.assert_close(dk.cpu()[vk], dkr[vk], rtol=5e-4, atol=1e-4)
    torch.testing.assert_close(dv.cpu()[vk], dvr[vk], rtol=5e-4, atol=1e-4)
    hidden = ~vq                                               # rows that see nothing: zero output, zero gradient
    if hidden.any():
        assert float(o.cpu().view(B, Sq, H, D)[hidden].abs().max()) == 0.0
        assert float(dq.cpu()[hidden].abs().max()) == 0.0


def test_fp32_attention_through_autograd_on_gpu(monkeypatch):
    """fp32 CUDA tensors through ``ops.block_attention`` (the autograd function the models call) take the fp32 kernels
    and give the CPU gradients."""
    from opentau_b200 import ops
    monkeypatch.setenv("OPENTAU_B200_F32_ATTN", "kernel")
    dev = torch.device("cuda:0")
    B, Sq, H, Hkv, D = 2, 70, 8, 2, 64
    _, _, _, qb, kb, qv, kv = _case(B, Sq, H, Hkv, D, 0, dev, seed=9)
    g = torch.Generator().manual_seed(3)
    q = torch.randn(B, Sq, H, D, generator=g)
    k = torch.randn(B, Sq, Hkv, D, generator=g)
    v = torch.randn(B, Sq, Hkv, D, generator=g)
    w = torch.randn(B, Sq, H * D, generator=g) * qv.cpu()[:, :, None]
    outs = []
    for device in ("cpu", dev):
        a, b_, c = (t.clone().to(device).requires_grad_(True) for t in (q, k, v))
        o = ops.block_attention(a, b_, c, qb.to(device), kb.to(device), qv.to(device), kv.to(device), D ** -0.5)
        (o * w.to(device)).sum().backward()
        outs.append((o.detach().cpu(), a.grad.cpu(), b_.grad.cpu(), c.grad.cpu()))
    (o_c, dq_c, dk_c, dv_c), (o_g, dq_g, dk_g, dv_g) = outs
    vq = qv.cpu()
    torch.testing.assert_close(o_g[vq], o_c[vq], rtol=5e-4, atol=5e-5)
    torch.testing.assert_close(dq_g[vq], dq_c[vq], rtol=5e-4, atol=1e-4)
    torch.testing.assert_close(dk_g[vq], dk_c[vq], rtol=5e-4, atol=1e-4)
    torch.testing.assert_close(dv_g[vq], dv_c[vq], rtol=5e-4, atol=1e-4)
