"""Training-side elementwise kernels (fused dropout + gated residual, masked flow-matching MSE, embedding gather /
scatter-add) against plain PyTorch fp32 statements of the same ops (run on a B200)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


@pytest.mark.parametrize("shape,gate_rows", [((4, 50, 1024), 1), ((3, 200, 2048), None), ((2, 7, 64), 7)])
def test_dropout_gated_residual_forward_and_backward(shape, gate_rows, dev):
    from opentau_b200 import ops
    from opentau_b200.ops import cuda_ops
    B, T, H = shape
    torch.manual_seed(1)
    x = torch.randn(B, T, H, device=dev).to(torch.bfloat16)
    y = torch.randn(B, T, H, device=dev).to(torch.bfloat16).requires_grad_(True)
    gate = None if gate_rows is None else torch.randn(B, gate_rows, H, device=dev).to(torch.bfloat16).requires_grad_(True)
    xr = x.clone().requires_grad_(True)
    p = 0.25
    out = ops.dropout_gated_residual(xr, y, gate, p, True)
    # the mask the kernel used, recovered from the kernel itself with x = 0, y = 1, no gate (same seed)
    seed = out.grad_fn.seed
    keep = cuda_ops.dropout_residual_fwd(torch.zeros_like(x), torch.ones_like(x), None, p, seed).float()
    kept = (keep != 0)
    assert abs(float(kept.float().mean()) - (1 - p)) < 0.02
    torch.testing.assert_close(keep[kept], torch.full_like(keep[kept], 1 / (1 - p)), rtol=1e-2, atol=1e-2)
    g = gate.float() if gate is not None else 1.0
    want = x.float() + g * (y.float() * keep)
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)
    dout = torch.randn_like(out)
    out.backward(dout)
    torch.testing.assert_close(xr.grad.float(), dout.float(), rtol=0, atol=0)
    torch.testing.assert_close(y.grad.float(), dout.float() * g * keep, rtol=2e-2, atol=2e-2)
    if gate is not None:
        dg = (dout.float() * y.float() * keep).view(B, gate_rows, T // gate_rows, H).sum(2)
        torch.testing.assert_close(gate.grad.float(), dg, rtol=3e-2, atol=3e-2 * float(dg.abs().max()))
    # a different call draws a different mask; eval mode is the plain residual
    out2 = ops.dropout_gated_residual(x, y.detach(), gate.detach() if gate is not None else None, p, True)
    assert not torch.equal(out2, out.detach())
    plain = ops.dropout_gated_residual(x, y.detach(), gate.detach() if gate is not None else None, p, False)
    torch.testing.assert_close(plain.float(), x.float() + g * y.float() if gate is None else
                               (x.float() + gate.float() * y.float()), rtol=2e-2, atol=2e-2)


def test_masked_mse_matches_reference_with_all_masks(dev):
    from opentau_b200 import ops
    from opentau_b200.ops import reference as ref
    torch.manual_seed(2)
    B, T, D = 6, 50, 32
    u = torch.randn(B, T, D, device=dev)
    v = torch.randn(B, T, D, device=dev, requires_grad=True)
    frozen = torch.rand(B, T, device=dev) < 0.2
    pad = torch.rand(B, T, device=dev) < 0.1
    real = torch.randint(5, D + 1, (B,), device=dev)
    loss, (s, c) = ops.flow_matching_masked_mse(u, v, frozen, pad, real, return_per_sample=True)
    vr = v.detach().clone().requires_grad_(True)
    want, (ws, wc) = ref.flow_matching_masked_mse(u, vr, frozen, pad, real, return_per_sample=True)
    torch.testing.assert_close(loss, want, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(s, ws, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(c, wc)
    (loss * 3.0).backward()
    (want * 3.0).backward()
    torch.testing.assert_close(v.grad, vr.grad, rtol=1e-5, atol=1e-7)
    # no masks at all
    l2 = ops.flow_matching_masked_mse(u, v.detach())
    torch.testing.assert_close(l2, ((u - v.detach()) ** 2).mean(), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("grad_dtype", [torch.bfloat16, torch.float32])
def test_embedding_gather_and_scatter_add(grad_dtype, dev):
    from opentau_b200 import ops
    torch.manual_seed(3)
    V, H = 1000, 256
    table = torch.nn.Parameter((torch.randn(V, H, device=dev) * 0.1).to(torch.bfloat16))
    ids = torch.randint(0, V, (4, 37), device=dev)
    ids[0, :5] = 7                                    # repeated ids: their rows must be summed
    ids[1, :3] = 0                                    # the padding row
    scale = 3.5
    out = ops.embedding(table, ids, scale, padding_idx=0)
    torch.testing.assert_close(out.float(), table.detach().float()[ids] * scale, rtol=1e-2, atol=1e-2)
    dout = torch.randn_like(out)
    want = torch.zeros(V, H, device=dev)
    want.index_add_(0, ids.reshape(-1), dout.float().reshape(-1, H) * scale)
    want[0] = 0
    # through autograd (.grad) ...
    out.backward(dout)
    torch.testing.assert_close(table.grad.float(), want, rtol=2e-2, atol=2e-2)
    # ... and straight into a flat gradient buffer of either dtype, accumulating on top of what is there
    table.grad = None
    table.main_grad = torch.ones(V, H, device=dev, dtype=grad_dtype)
    ops.embedding(table, ids, scale, padding_idx=0).backward(dout)
    assert table.grad is None
    torch.testing.assert_close(table.main_grad.float(), want + 1.0, rtol=2e-2, atol=3e-2)
    # run twice: bitwise the same (fixed summation order, no atomics)
    a = torch.zeros(V, H, device=dev)
    b = torch.zeros(V, H, device=dev)
    from opentau_b200.ops import cuda_ops
    cuda_ops.embed_bwd(dout, ids, a, scale, 0)
    cuda_ops.embed_bwd(dout, ids, b, scale, 0)
    assert torch.equal(a, b)


@pytest.mark.parametrize("with_bias,into_main_grad", [(True, False), (False, True)])
def test_vocabulary_tiled_cross_entropy_head(with_bias, into_main_grad, dev, monkeypatch):
    """The CE head over several vocabulary tiles (no rows x vocabulary tensor in either direction) equals the fp32
    statement; also with the weight gradient accumulated straight into a flat gradient buffer."""
    from opentau_b200 import ops
    from opentau_b200.ops import cuda_ops
    monkeypatch.setattr(cuda_ops, "CE_VOCAB_TILE", 256)
    torch.manual_seed(4)
    R, H, V = 300, 128, 1000                           # tiles of 256, 256, 256 and 232 columns
    h = (torch.randn(R, H, device=dev) * 0.5).to(torch.bfloat16).requires_grad_(True)
    w = torch.nn.Parameter((torch.randn(V, H, device=dev) * 0.2).to(torch.bfloat16))
    b = torch.nn.Parameter((torch.randn(V, device=dev) * 0.1).to(torch.bfloat16)) if with_bias else None
    labels = torch.randint(0, V, (R,), device=dev)
    labels[:4] = torch.tensor([0, 255, 256, V - 1], device=dev)      # tile borders
    if into_main_grad:
        w.main_grad = torch.full((V, H), 0.5, device=dev, dtype=torch.bfloat16)
    loss = ops.linear_cross_entropy(h, w, b, labels)
    hr, wr = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    br = b.detach().float().requires_grad_(True) if with_bias else None
    want = torch.nn.functional.cross_entropy(torch.nn.functional.linear(hr, wr, br), labels, reduction="none")
    torch.testing.assert_close(loss, want, rtol=2e-2, atol=2e-2)
    wts = torch.rand(R, device=dev)
    (loss * wts).sum().backward()
    (want * wts).sum().backward()
    torch.testing.assert_close(h.grad.float(), hr.grad, rtol=5e-2, atol=2e-2)
    if into_main_grad:
        assert w.grad is None
        torch.testing.assert_close(w.main_grad.float() - 0.5, wr.grad, rtol=5e-2, atol=3e-2)
    else:
        torch.testing.assert_close(w.grad.float(), wr.grad, rtol=5e-2, atol=3e-2)
    if with_bias:
        torch.testing.assert_close(b.grad.float(), br.grad, rtol=5e-2, atol=3e-2)


@pytest.mark.parametrize("grid", [(16, 16), (13, 23), (32, 20), (7, 7)])
def test_position_table_resample_matches_bicubic_interpolate(grid, dev):
    """Native-resolution inputs: the 16 x 16 SigLIP position table resampled to the image's patch grid equals
    ``F.interpolate(mode="bicubic", align_corners=False)``."""
    from opentau_b200.ops import cuda_ops
    torch.manual_seed(5)
    g, d = 16, 96
    tab = torch.randn(g * g, d, device=dev)
    gh, gw = grid
    got = cuda_ops.pos_resample(tab, gh, gw)
    want = torch.nn.functional.interpolate(tab.view(1, g, g, d).permute(0, 3, 1, 2), size=(gh, gw), mode="bicubic",
                                           align_corners=False).permute(0, 2, 3, 1).reshape(gh * gw, d)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)


def test_native_resolution_image_through_the_vision_tower(dev):
    """A 180 x 320 image (not a patch multiple, not the config grid) is padded to patches and embedded with the
    resampled position table; the tower's output matches the CPU fp32 tower."""
    import sys, os
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from opentau_b200.models.siglip import SiglipConfig, SiglipVisionModel
    torch.manual_seed(6)
    cfg = SiglipConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                       patch_size=14, image_size=224)
    cpu = SiglipVisionModel(cfg).eval()
    gpu = SiglipVisionModel(cfg).eval()
    gpu.load_state_dict(cpu.state_dict())
    gpu = gpu.to(dev).to(torch.bfloat16)
    x = torch.rand(2, 3, 180, 320) * 2 - 1
    with torch.no_grad():
        want = cpu(x)
        got = gpu(x.to(dev).to(torch.bfloat16))
    assert got.shape == want.shape == (2, 13 * 23, 128)
    torch.testing.assert_close(got.float().cpu(), want, rtol=5e-2, atol=5e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,T,H,W,C,L,k", [(2, 4, 16, 16, 256, 5, 9), (1, 3, 5, 7, 64, 3, 3), (2, 2, 6, 4, 96, 1, 5),
                                           (1, 6, 4, 4, 40, 5, 3)])
def test_stss_window_correlation_kernels_match_the_dense_evaluation(dtype, B, T, H, W, C, L, k):
    """Forward and backward of the space-time window correlation against the unfold + einsum evaluation on the CPU in
    fp32: clamped frame offsets (a frame is its own neighbour at the ends, so a feature is source and target of the
    same product), zeros outside the image, a head width that is not a power of two, L = 1."""
    from opentau_b200.ops import stss
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(B * 100 + C + L)
    x = torch.nn.functional.normalize(torch.randn(B, T, H * W, C, generator=g), dim=-1)
    w = torch.randn(B, T, H * W, L, k * k, generator=g)
    xc = x.to(dtype).float().detach().clone().requires_grad_(True)
    ref = stss.dense_window_correlation(xc, T, H, W, L, k)
    (ref * w).sum().backward()
    xg = x.to(dtype).to(dev).detach().clone().requires_grad_(True)
    assert stss.native_supported(xg)
    out = stss.local_window_correlation(xg, T, H, W, L, k)
    (out.float() * w.to(dev)).sum().backward()
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=1e-2)
    torch.testing.assert_close(out.float().cpu(), ref.detach(), **tol)
    gtol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=0.15)
    torch.testing.assert_close(xg.grad.float().cpu(), xc.grad, **gtol)


def test_seq_concat_kernel_matches_cat_forward_and_backward(dev):
    """Cached keys followed by new keys: a layer view of a (L, B, S, H, D) cache with spare room (strided batch) and a
    strided slice of a fused projection, against ``torch.cat``; gradients are the slices of the incoming gradient."""
    from opentau_b200 import ops
    from opentau_b200.ops import cuda_ops
    torch.manual_seed(0)
    cache = torch.randn(3, 4, 40, 2, 64, device=dev).to(torch.bfloat16)
    a = cache[1][:, :33]                                         # (4, 33, 2, 64): batch stride 40 * 128
    fused_qkv = torch.randn(4, 7, 6, 64, device=dev).to(torch.bfloat16)
    c = fused_qkv[:, :, 4:].detach().requires_grad_(True)        # (4, 7, 2, 64): row stride 6 * 64
    assert cuda_ops.seq_concat_supported(a, c)
    out = ops.seq_concat(a, c)
    ref = torch.cat([a, c.detach()], dim=1)
    assert out.shape == (4, 40, 2, 64) and torch.equal(out, ref)
    w = torch.randn_like(out)
    (out.float() * w.float()).sum().backward()
    torch.testing.assert_close(c.grad.float(), w[:, 33:].float())
    odd = torch.randn(4, 7, 1, 60, device=dev).to(torch.bfloat16)   # 60 elements per row: not a multiple of 8 -> cat
    assert not cuda_ops.seq_concat_supported(odd, odd) and ops.seq_concat(odd, odd).shape == (4, 14, 1, 60)
    assert torch.equal(ops.seq_concat(a.float().cpu(), c.detach().float().cpu()), ref.float().cpu())


def test_zero_fill_through_memset(dev):
    from opentau_b200.ops import cuda_ops
    t = torch.randn(3, 1000, 7, device=dev, dtype=torch.bfloat16)
    view = t[1]
    cuda_ops.zero_(view)                                  # a dense slice: only its bytes are cleared
    assert float(view.abs().sum()) == 0.0 and float(t[0].abs().sum()) > 0 and float(t[2].abs().sum()) > 0
    strided = t[:, ::2]
    cuda_ops.zero_(strided)                               # not dense: the element-wise fallback
    assert float(strided.abs().sum()) == 0.0 and float(t[0, 1::2].abs().sum()) > 0
    big = torch.ones(64 << 20, device=dev, dtype=torch.bfloat16)
    cuda_ops.zero_(big)
    assert float(big.float().sum()) == 0.0
