"""sm_100a kernels against plain PyTorch fp32 references of the same op (run on a B200)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def _ref_gemm(a, b, layout):
    a, b = a.float(), b.float()
    if layout == "nt":
        return a @ b.t()
    if layout == "nn":
        return a @ b
    return a.t() @ b


def _operands(layout, M, N, K, dev):
    g = torch.Generator(device="cpu").manual_seed(M * 7 + N * 3 + K)
    mk = lambda *s: (torch.randn(*s, generator=g) * 0.5).to(torch.bfloat16).to(dev)  # noqa: E731
    if layout == "nt":
        return mk(M, K), mk(N, K)
    if layout == "nn":
        return mk(M, K), mk(K, N)
    return mk(K, M), mk(K, N)


@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (200, 264, 136), (1000, 2048, 1024),
                                   (50, 1024, 2048), (384, 64, 512), (130, 128, 72)])
@pytest.mark.parametrize("bn", [0, 64, 128, 256, 512])        # 512: the CTA-pair kernel (256 x 256 tiles on two SMs)
def test_gemm_layouts(layout, shape, bn, dev):
    from opentau_b200.ops import cuda_ops
    M, N, K = shape
    if layout == "tn" and M % 8:
        pytest.skip("MN-major A needs M % 8 == 0")
    a, b = _operands(layout, M, N, K, dev)
    out = cuda_ops.gemm(a, b, layout, bn=bn)
    cuda_ops.check_status()
    ref = _ref_gemm(a, b, layout)
    err = (out.float() - ref).abs().max().item()
    tol = 2e-2 * max(1.0, ref.abs().max().item())
    assert err <= tol, f"{layout} {shape} bn={bn}: max err {err} (tol {tol})"


def test_gemm_epilogues(dev):
    from opentau_b200.ops import cuda_ops
    M, N, K = 300, 512, 320
    a, b = _operands("nt", M, N, K, dev)
    bias = torch.randn(N, device=dev).to(torch.bfloat16)
    res = torch.randn(M, N, device=dev).to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    out = cuda_ops.gemm(a, b, "nt", bias=bias, residual=res)
    torch.testing.assert_close(out.float(), ref + bias.float() + res.float(), rtol=2e-2, atol=8e-2)
    out32 = cuda_ops.gemm(a, b, "nt", bias=bias.float(), out_dtype=torch.float32)
    torch.testing.assert_close(out32, ref + bias.float(), rtol=1e-3, atol=1e-2)
    acc = torch.ones(M, N, device=dev, dtype=torch.bfloat16)
    cuda_ops.gemm(a, b, "nt", out=acc, accumulate=True)
    torch.testing.assert_close(acc.float(), ref + 1.0, rtol=2e-2, atol=8e-2)
    g = cuda_ops.gemm(a, b, "nt", bias=bias, act="gelu_tanh")
    torch.testing.assert_close(g.float(), torch.nn.functional.gelu(ref + bias.float(), approximate="tanh"),
                               rtol=2e-2, atol=8e-2)
    cuda_ops.check_status()


@pytest.mark.parametrize("shape", [(51, 1024, 2048), (1, 256, 64), (64, 4096, 1024), (100, 1152, 4304), (128, 128, 128),
                                   (211, 5120, 1000), (588, 1152, 1152), (300, 200, 72)])
@pytest.mark.parametrize("splits", [0, 1, 2, 3, 4, 7, 8])
def test_skinny_gemm_matches_fp32(shape, splits, dev):
    """Weight-streaming split-K kernel: all token-tile widths, several token chunks, ragged N and K, every cluster size."""
    from opentau_b200.ops import cuda_ops
    M, N, K = shape
    a, b = _operands("nt", M, N, K, dev)
    out = cuda_ops.gemm(a, b, "nt", splits=splits or (0 if cuda_ops.use_skinny("nt", M, N, False, 0) else 2))
    again = cuda_ops.gemm(a, b, "nt", splits=splits or (0 if cuda_ops.use_skinny("nt", M, N, False, 0) else 2))
    cuda_ops.check_status()
    ref = _ref_gemm(a, b, "nt")
    err = (out.float() - ref).abs().max().item()
    tol = 2e-2 * max(1.0, ref.abs().max().item())
    assert err <= tol, f"{shape} splits={splits}: max err {err} (tol {tol})"
    assert torch.equal(out, again)                    # the cluster reduction has a fixed order


@pytest.mark.parametrize("splits", [1, 4])
def test_skinny_gemm_epilogues(splits, dev):
    from opentau_b200.ops import cuda_ops
    M, N, K = 51, 520, 320
    a, b = _operands("nt", M, N, K, dev)
    bias = torch.randn(N, device=dev).to(torch.bfloat16)
    res = torch.randn(M, N, device=dev).to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    out = cuda_ops.gemm(a, b, "nt", bias=bias, residual=res, splits=splits)
    torch.testing.assert_close(out.float(), ref + bias.float() + res.float(), rtol=2e-2, atol=8e-2)
    out32 = cuda_ops.gemm(a, b, "nt", bias=bias.float(), out_dtype=torch.float32, splits=splits)
    torch.testing.assert_close(out32, ref + bias.float(), rtol=1e-3, atol=1e-2)
    g = cuda_ops.gemm(a, b, "nt", bias=bias, act="gelu_tanh", splits=splits)
    torch.testing.assert_close(g.float(), torch.nn.functional.gelu(ref + bias.float(), approximate="tanh"),
                               rtol=2e-2, atol=8e-2)
    cuda_ops.check_status()


@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
@pytest.mark.parametrize("splits", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("M", [51, 200])
def test_skinny_gemm_glu(act, splits, M, dev):
    from opentau_b200.ops import cuda_ops, prims
    K, I = 256, 384
    x = (torch.randn(M, K) * 0.5).to(torch.bfloat16).to(dev)
    w = (torch.randn(2 * I, K) * 0.1).to(torch.bfloat16).to(dev)
    gu, h = cuda_ops.gemm(x, w, "nt", glu=act, splits=splits)
    gu_ref = (x.float() @ w.float().t()).to(torch.bfloat16)
    torch.testing.assert_close(gu.float(), gu_ref.float(), rtol=2e-2, atol=3e-2)
    h_ref = prims.glu_fwd(gu_ref.cpu().float(), act).to(dev)
    torch.testing.assert_close(h.float(), h_ref, rtol=3e-2, atol=3e-2)
    h_only = cuda_ops.gemm(x, w, "nt", glu=act, store_out=False, splits=splits)
    torch.testing.assert_close(h_only.float(), h.float())
    cuda_ops.check_status()


@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
def test_gemm_glu_epilogue(act, dev):
    from opentau_b200.ops import cuda_ops, prims
    M, K, I = 260, 256, 384
    x = (torch.randn(M, K) * 0.5).to(torch.bfloat16).to(dev)
    w = (torch.randn(2 * I, K) * 0.1).to(torch.bfloat16).to(dev)
    gu, h = cuda_ops.gemm(x, w, "nt", glu=act)
    gu_ref = (x.float() @ w.float().t()).to(torch.bfloat16)
    torch.testing.assert_close(gu.float(), gu_ref.float(), rtol=2e-2, atol=3e-2)
    h_ref = prims.glu_fwd(gu_ref.cpu().float(), act).to(dev)
    torch.testing.assert_close(h.float(), h_ref, rtol=3e-2, atol=3e-2)
    h_only = cuda_ops.gemm(x, w, "nt", glu=act, store_out=False)
    torch.testing.assert_close(h_only.float(), h.float())
    h2 = cuda_ops.glu_fwd(gu, act)
    torch.testing.assert_close(h2.float(), h.float(), rtol=2e-2, atol=2e-2)
    dh = torch.randn(M, I, device=dev).to(torch.bfloat16)
    dgu = cuda_ops.glu_bwd(gu, dh, act)
    dgu_ref = prims.glu_bwd(gu.cpu().float(), dh.cpu().float(), act)
    torch.testing.assert_close(dgu.cpu().float(), dgu_ref, rtol=3e-2, atol=3e-2)
    cuda_ops.check_status()


@pytest.mark.parametrize("H", [64, 256, 1024, 1152, 2048, 5120])
@pytest.mark.parametrize("mode", ["plain1", "plain0", "noweight"])
def test_rms_norm_kernels(H, mode, dev):
    from opentau_b200.ops import cuda_ops, prims
    R = 77
    x = torch.randn(R, H, device=dev).to(torch.bfloat16)
    w = (torch.randn(H, device=dev) * 0.1).to(torch.bfloat16) if mode != "noweight" else None
    unit = mode == "plain1"
    y, rstd = cuda_ops.rms_fwd(x, w, 1e-6, unit)
    yr, rr = prims.rms_fwd(x.cpu().float(), None if w is None else w.cpu().float(), 1e-6, unit)
    torch.testing.assert_close(y.cpu().float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(rstd.cpu(), rr, rtol=1e-4, atol=1e-5)
    dy = torch.randn(R, H, device=dev).to(torch.bfloat16)
    dx, dw = cuda_ops.rms_bwd(dy, x, w, rstd, unit)
    dxr, dwr = prims.rms_bwd(dy.cpu().float(), x.cpu().float(), None if w is None else w.cpu().float(), rr, unit)
    torch.testing.assert_close(dx.cpu().float(), dxr, rtol=3e-2, atol=3e-2)
    if w is not None:
        torch.testing.assert_close(dw.cpu().float(), dwr, rtol=3e-2, atol=1e-1)


@pytest.mark.parametrize("per_token", [True, False])
def test_ada_rms_kernels(per_token, dev):
    from opentau_b200.ops import cuda_ops, prims
    B, S, H = 3, 10, 1024
    x = torch.randn(B, S, H, device=dev).to(torch.bfloat16)
    mod = (torch.randn(B, S, 3 * H, device=dev) * 0.3).to(torch.bfloat16)
    if not per_token:
        mod = mod[:, 0].contiguous()
    y, rstd = cuda_ops.ada_rms_fwd(x, mod, 1e-6)
    yr, rr = prims.ada_rms_fwd(x.cpu().float(), mod.cpu().float(), 1e-6)
    torch.testing.assert_close(y.cpu().float(), yr, rtol=2e-2, atol=3e-2)
    dy = torch.randn(B, S, H, device=dev).to(torch.bfloat16)
    dx, dsc, dsh = cuda_ops.ada_rms_bwd(dy, x, mod, rstd)
    dxr, dscr, dshr = prims.ada_rms_bwd(dy.cpu().float(), x.cpu().float(), mod.cpu().float(), rr)
    torch.testing.assert_close(dx.cpu().float(), dxr, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(dsc.cpu().float(), dscr, rtol=3e-2, atol=1e-1)
    torch.testing.assert_close(dsh.cpu().float(), dshr, rtol=3e-2, atol=1e-1)


def test_layer_norm_kernel(dev):
    from opentau_b200.ops import cuda_ops, prims
    x = torch.randn(50, 1152, device=dev).to(torch.bfloat16)
    w = torch.randn(1152, device=dev).to(torch.bfloat16)
    b = torch.randn(1152, device=dev).to(torch.bfloat16)
    y, mean, rstd = cuda_ops.ln_fwd(x, w, b, 1e-6)
    yr, mr, rr = prims.ln_fwd(x.cpu().float(), w.cpu().float(), b.cpu().float(), 1e-6)
    torch.testing.assert_close(y.cpu().float(), yr, rtol=2e-2, atol=3e-2)
    torch.testing.assert_close(mean.cpu(), mr, rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("D", [64, 72])     # 72: Qwen3-VL vision heads (8-byte accesses)
def test_rope_kernel_strided(dev, D):
    from opentau_b200 import ops
    from opentau_b200.ops import cuda_ops
    B, S, H = 2, 33, 4
    qkv = torch.randn(B, S, (H + 2) * D, device=dev).to(torch.bfloat16)
    q = qkv[..., :H * D].unflatten(-1, (H, D))
    pos = torch.arange(S, device=dev)[None].expand(B, -1)
    cos, sin = ops.rope_angles(pos, D, 10000.0)
    y = cuda_ops.rope_fwd(q, cos, sin)
    yr = ops.ref.apply_rope(q.float(), cos, sin)
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    back = cuda_ops.rope_fwd(y, cos, sin, inverse=True)
    torch.testing.assert_close(back.float(), q.float(), rtol=3e-2, atol=3e-2)


def test_linear_ce_kernels(dev):
    from opentau_b200.ops import cuda_ops, prims
    R, H, V = 96, 256, 2048
    h = torch.randn(R, H, device=dev).to(torch.bfloat16)
    w = (torch.randn(V, H, device=dev) * 0.05).to(torch.bfloat16)
    b = (torch.randn(V, device=dev) * 0.1).to(torch.bfloat16)
    labels = torch.randint(0, V, (R,), device=dev)
    loss, lse = cuda_ops.linear_ce_fwd(h, w, b, labels)
    lr_, lser = prims.linear_ce_fwd(h.cpu().float(), w.cpu().float(), b.cpu().float(), labels.cpu())
    torch.testing.assert_close(loss.cpu(), lr_, rtol=1e-2, atol=2e-2)
    dloss = torch.rand(R, device=dev)
    dh, dw, db = cuda_ops.linear_ce_bwd(dloss, h, w, b, labels, lse)
    dhr, dwr, dbr = prims.linear_ce_bwd(dloss.cpu(), h.cpu().float(), w.cpu().float(), b.cpu().float(), labels.cpu(), lser)
    torch.testing.assert_close(dh.cpu().float(), dhr, rtol=5e-2, atol=2e-2)
    torch.testing.assert_close(dw.cpu().float(), dwr, rtol=5e-2, atol=3e-2)
    torch.testing.assert_close(db.cpu().float(), dbr, rtol=5e-2, atol=3e-2)


def test_adamw_and_clip_kernels(dev):
    from opentau_b200.ops import cuda_ops
    from opentau_b200.ops import reference as ref
    n = 100_003
    p = torch.randn(n, device=dev)
    g = torch.randn(n, device=dev).to(torch.bfloat16)
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    p16 = torch.empty(n, device=dev, dtype=torch.bfloat16)
    pr, mr, vr = p.clone().cpu(), m.clone().cpu(), v.clone().cpu()
    scale = torch.tensor([0.5, 0.0], device=dev)
    for step in (1, 2, 3):
        cuda_ops.adamw(p, g, m, v, p16, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01, step=step, scale=scale)
        ref.adamw_flat(pr, g.cpu(), mr, vr, None, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01,
                       step=step, grad_scale=0.5)
    torch.testing.assert_close(p.cpu(), pr, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(p16.cpu().float(), pr, rtol=1e-2, atol=1e-2)
    partial = torch.zeros(1024, device=dev)
    cuda_ops.sumsq_partials(g, partial)
    torch.testing.assert_close(partial.sum().cpu(), g.float().pow(2).sum().cpu(), rtol=1e-4, atol=1e-2)
    out = torch.zeros(2, device=dev)
    cuda_ops.clip_coef(partial, 0.25, 1.0, out)
    norm = g.float().pow(2).sum().sqrt().item() * 0.25
    assert abs(out[1].item() - norm) / norm < 1e-4
    assert abs(out[0].item() - 0.25 * min(1.0, 1.0 / (norm + 1e-6))) < 1e-6


@pytest.mark.parametrize("offset,grad_dtype,with_p16", [(0, torch.bfloat16, True), (1, torch.bfloat16, True),
                                                          (0, torch.float32, False), (4, torch.float32, True)])
def test_adamw_vector_and_scalar_paths_agree_with_reference(dev, offset, grad_dtype, with_p16):
    """Aligned buffers take the 8-wide kernel plus a scalar tail; views that start off a 16-byte boundary take the
    scalar kernel for everything.  Both must give the fp32 reference."""
    from opentau_b200.ops import cuda_ops
    from opentau_b200.ops import reference as ref
    n = 65_536 + 5
    base = [torch.randn(n + 8, device=dev) for _ in range(2)]
    p = base[0][offset:offset + n]
    g = base[1].to(grad_dtype)[offset:offset + n]
    m, v = torch.zeros(n + 8, device=dev)[offset:offset + n], torch.zeros(n + 8, device=dev)[offset:offset + n]
    p16 = torch.empty(n + 8, device=dev, dtype=torch.bfloat16)[offset:offset + n] if with_p16 else None
    pr, mr, vr = p.clone().cpu(), m.clone().cpu(), v.clone().cpu()
    guard = base[0][offset + n:].clone()
    for step in (1, 2):
        cuda_ops.adamw(p, g, m, v, p16, lr=3e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
        ref.adamw_flat(pr, g.cpu(), mr, vr, None, lr=3e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
    torch.testing.assert_close(p.cpu(), pr, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(m.cpu(), mr, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(v.cpu(), vr, rtol=1e-4, atol=1e-7)
    if with_p16:
        torch.testing.assert_close(p16.cpu().float(), pr, rtol=1e-2, atol=1e-2)
    assert torch.equal(base[0][offset + n:], guard)            # nothing written past the end


@pytest.mark.parametrize("rows,H", [(1000, 1152), (37, 64), (600, 4096)])
def test_layer_norm_backward_kernel(dev, rows, H):
    """dx, dw, db of the native LayerNorm backward against autograd on the fp32 statement of the same op."""
    from opentau_b200.ops import cuda_ops
    torch.manual_seed(rows + H)
    x = (torch.randn(rows, H, device=dev) * 2 + 0.5).to(torch.bfloat16)
    w = (torch.randn(H, device=dev) * 0.3 + 1).to(torch.bfloat16)
    b = (torch.randn(H, device=dev) * 0.1).to(torch.bfloat16)
    dy = torch.randn(rows, H, device=dev).to(torch.bfloat16)
    y, mean, rstd = cuda_ops.ln_fwd(x, w, b, 1e-6)
    dx, dw, db = cuda_ops.ln_bwd(dy, x, w, mean, rstd)
    xr = x.float().cpu().requires_grad_(True)
    wr, br = w.float().cpu().requires_grad_(True), b.float().cpu().requires_grad_(True)
    yr = torch.nn.functional.layer_norm(xr, (H,), wr, br, 1e-6)
    yr.backward(dy.float().cpu())
    torch.testing.assert_close(y.float().cpu(), yr.detach(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(dx.float().cpu(), xr.grad, rtol=2e-2, atol=2e-2)
    scale = max(1.0, rows ** 0.5)
    torch.testing.assert_close(dw.float().cpu() / scale, wr.grad / scale, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(db.float().cpu() / scale, br.grad / scale, rtol=2e-2, atol=2e-2)
    assert dx.dtype == x.dtype and dw.shape == (H,) and db.shape == (H,)


def test_resize_pad_kernel(dev):
    from opentau_b200 import ops
    from opentau_b200.ops import cuda_ops
    img = torch.rand(2, 3, 120, 200, device=dev)
    out = cuda_ops.resize_with_pad(img, 224, 224, 0.0)
    ref = ops.ref.resize_with_pad(img.cpu(), 224, 224, 0.0)
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-4)


def test_native_libraries_are_loaded(dev):
    from opentau_b200.ops import _lib, cuda_ops
    a = torch.randn(128, 64, device=dev).to(torch.bfloat16)
    cuda_ops.gemm(a, a, "nt")
    with open("/proc/self/maps") as f:
        maps = f.read()
    assert "libotb_gemm_tcgen05.so" in maps
    assert any("gemm_tcgen05" in p for p in _lib.loaded_libraries())


@pytest.mark.parametrize("H,Hkv,D,norm", [(8, 1, 256, False), (16, 8, 128, True), (4, 2, 72, True), (2, 2, 64, False)])
def test_qkv_post_matches_unfused_ops(H, Hkv, D, norm, dev):
    """split + qk-norm + rotation + strided K/V store in one launch == rms_norm, rope and copies done separately."""
    from opentau_b200 import ops
    from opentau_b200.models.layers import RMSNorm
    B, T, P = 2, 51, 37
    torch.manual_seed(0)
    qkv = torch.randn(B, T, (H + 2 * Hkv) * D, device=dev).to(torch.bfloat16)
    pos = torch.arange(T, device=dev)[None].expand(B, -1) + 5
    cos, sin = ops.rope_angles(pos, D, 10000.0)
    qn = kn = None
    if norm:
        qn, kn = RMSNorm(D, 1e-6, False).to(dev).to(torch.bfloat16), RMSNorm(D, 1e-6, False).to(dev).to(torch.bfloat16)
        with torch.no_grad():
            qn.weight.add_(torch.randn_like(qn.weight) * 0.1), kn.weight.add_(torch.randn_like(kn.weight) * 0.1)
    with torch.no_grad():
        q, k, v = qkv.split([H * D, Hkv * D, Hkv * D], dim=-1)
        q, k, v = q.unflatten(-1, (H, D)), k.unflatten(-1, (Hkv, D)), v.unflatten(-1, (Hkv, D))
        if norm:
            q, k = qn(q)[0], kn(k)[0]
        want_q, want_k = ops.rope(q, cos, sin), ops.rope(k, cos, sin)
        got_q, got_k, got_v = ops.qkv_post(qkv, H, Hkv, D, qn, kn, cos, sin)
        kbuf = torch.zeros(B, P + T + 3, Hkv, D, device=dev, dtype=torch.bfloat16)
        vbuf = torch.zeros_like(kbuf)
        ops.qkv_post(qkv, H, Hkv, D, qn, kn, cos, sin, kbuf[:, P:P + T], vbuf[:, P:P + T])
    torch.testing.assert_close(got_q.float(), want_q.float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(got_k.float(), want_k.float(), atol=2e-2, rtol=2e-2)
    assert torch.equal(got_v, v)
    assert torch.equal(kbuf[:, P:P + T], got_k) and torch.equal(vbuf[:, P:P + T], got_v)
    assert float(kbuf[:, :P].abs().sum()) == 0 and float(kbuf[:, P + T:].abs().sum()) == 0


@pytest.mark.parametrize("per_token", [False, True])
def test_gated_residual_native(per_token, dev):
    from opentau_b200 import ops
    B, T, H = 3, 51, 1024
    x, y = (torch.randn(B, T, H, device=dev).to(torch.bfloat16) for _ in range(2))
    mod = torch.randn(B, T if per_token else 1, 3 * H, device=dev).to(torch.bfloat16)
    gate = mod[..., 2 * H:]                                    # a strided slice, as the adaptive norm hands it out
    with torch.no_grad():
        got = ops.gated_residual(x, y, gate)
    want = x.float() + y.float() * gate.float()
    torch.testing.assert_close(got.float(), want, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("per_token", [False, True])
@pytest.mark.parametrize("splits", [0, 1, 4])
def test_skinny_gemm_gated_residual_epilogue(per_token, splits, dev):
    """out = residual + gate * (x @ W^T): the adaptive-norm gate of a residual branch applied in the projection."""
    from opentau_b200 import ops
    from opentau_b200.ops import cuda_ops
    B, T, K, N = 2, 51, 512, 1024
    x = (torch.randn(B, T, K, device=dev) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
    res = torch.randn(B, T, N, device=dev).to(torch.bfloat16)
    mod = torch.randn(B, T if per_token else 1, 3 * N, device=dev).to(torch.bfloat16)
    gate = mod[..., 2 * N:]
    want = res.float() + gate.float() * (x.float() @ w.float().t())
    g2 = gate.reshape(-1, N)
    got = cuda_ops.gemm(x.view(B * T, K), w, "nt", residual=res.view(B * T, N), gate=g2, splits=splits)
    torch.testing.assert_close(got.float().view(B, T, N), want, atol=6e-2, rtol=3e-2)
    with torch.no_grad():
        via_ops = ops.linear_gated_residual(x, w, None, res, gate)
    torch.testing.assert_close(via_ops.float(), want, atol=6e-2, rtol=3e-2)
    wgu = (torch.randn(2 * 768, K, device=dev) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(K, 768, device=dev) * 0.05).to(torch.bfloat16)
    resk = torch.randn(B, T, K, device=dev).to(torch.bfloat16)
    modk = torch.randn(B, T if per_token else 1, 3 * K, device=dev).to(torch.bfloat16)
    gk = modk[..., 2 * K:]
    with torch.no_grad():
        fused = ops.gated_mlp_gated_residual(x, wgu, wd, "silu", resk, gk)
        plain = ops.gated_residual(resk, ops.gated_mlp(x, wgu, wd, "silu"), gk)
    torch.testing.assert_close(fused.float(), plain.float(), atol=6e-2, rtol=3e-2)
    cuda_ops.check_status()


def test_flow_matching_kernels(dev):
    """Time embedding, flow interpolation and the Euler step against their fp32 statements."""
    from opentau_b200 import ops
    B, T, D = 3, 51, 32
    time = torch.rand(B, T, device=dev)
    for dim, dt_ in ((1024, torch.float32), (256, torch.bfloat16)):
        got = ops.sinusoidal_time_embedding(time, dim, 4e-3, 4.0, out_dtype=dt_)
        want = ops.ref.sinusoidal_time_embedding(time.cpu(), dim, 4e-3, 4.0)
        assert got.dtype == dt_ and got.shape == (B, T, dim)
        # the largest angle is 2 pi / 4e-3 ~ 1571 rad: fp32 argument rounding bounds the error near 1e-4
        torch.testing.assert_close(got.float().cpu(), want, atol=1e-2 if dt_ == torch.bfloat16 else 2e-3, rtol=0)
    a, n = torch.randn(B, T, D, device=dev), torch.randn(B, T, D, device=dev)
    x_t, u_t = ops.flow_interpolate(a, n, time)
    wx, wu = ops.ref.flow_interpolate(a, n, time)
    torch.testing.assert_close(x_t, wx), torch.testing.assert_close(u_t, wu)
    frozen = torch.zeros(B, T, dtype=torch.bool, device=dev)
    frozen[:, :7] = True
    prefix = torch.randn(B, T, D, device=dev)
    for v in (torch.randn(B, T, D, device=dev), torch.randn(B, T, D, device=dev).to(torch.bfloat16)):
        x0 = torch.randn(B, T, D, device=dev)
        want = torch.where(frozen[:, :, None], prefix, x0 + (-0.1) * v.float())
        with torch.no_grad():
            got = ops.euler_step(x0.clone(), v, -0.1, frozen, prefix)
            plain = ops.euler_step(x0.clone(), v, -0.1)
        torch.testing.assert_close(got, want), torch.testing.assert_close(plain, x0 + (-0.1) * v.float())


@pytest.mark.parametrize("pix_dtype,out_dtype", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32)])
def test_patch_embed_kernel(pix_dtype, out_dtype, dev):
    """Fused gather + fp32 product + bias + position table against the unfold + linear statement, with gradients."""
    from opentau_b200 import ops
    B, C, H, W, p, N = 3, 3, 56, 42, 14, 200
    torch.manual_seed(0)
    pix = (torch.rand(B, C, H, W, device=dev) * 2 - 1).to(pix_dtype)
    w = (torch.randn(N, C, p, p, device=dev) * 0.05).requires_grad_(True)
    b = torch.randn(N, device=dev).requires_grad_(True)
    pos = torch.randn((H // p) * (W // p), N, device=dev).requires_grad_(True)
    got = ops.patch_embed(pix, w, b, pos, p, out_dtype)
    x = pix.float().view(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5).reshape(B, -1, C * p * p)
    w2, b2, pos2 = (t.detach().clone().requires_grad_(True) for t in (w, b, pos))
    want = torch.nn.functional.linear(x, w2.view(N, -1), b2) + pos2
    assert got.dtype == out_dtype and got.shape == want.shape
    torch.testing.assert_close(got.float(), want, atol=2e-2 if out_dtype == torch.bfloat16 else 1e-4, rtol=1e-2)
    g = torch.randn_like(want)
    got.backward(g.to(out_dtype))
    want.backward(g.to(out_dtype).float())
    torch.testing.assert_close(w.grad, w2.grad, atol=1e-3, rtol=1e-3)
    torch.testing.assert_close(b.grad, b2.grad, atol=1e-3, rtol=1e-3)
    torch.testing.assert_close(pos.grad, pos2.grad, atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
@pytest.mark.parametrize("shape", [(2048, 2048, 512), (1504, 1288, 328), (4096, 1024, 2048), (520, 264, 72)])
def test_cta_pair_gemm_epilogues(layout, shape, dev):
    """The CTA-pair kernel (tcgen05 cta_group::2, each CTA loads half of the B tile) on full, ragged and tiny
    problems, with the residual / bias / accumulate epilogues; run twice: bitwise identical."""
    from opentau_b200.ops import cuda_ops
    M, N, K = shape
    a, b = _operands(layout, M, N, K, dev)
    want = _ref_gemm(a, b, layout)
    got = cuda_ops.gemm(a, b, layout, bn=512)
    torch.testing.assert_close(got.float(), want, rtol=2e-2, atol=2e-2 * float(want.abs().max()))
    assert torch.equal(got, cuda_ops.gemm(a, b, layout, bn=512))
    bias = torch.randn(N, device=dev).to(torch.bfloat16)
    res = torch.randn(M, N, device=dev).to(torch.bfloat16)
    got2 = cuda_ops.gemm(a, b, layout, bias=bias, residual=res, bn=512)
    torch.testing.assert_close(got2.float(), want + bias.float() + res.float(), rtol=2e-2,
                               atol=2e-2 * float(want.abs().max()))
    acc = torch.ones(M, N, device=dev, dtype=torch.bfloat16)
    cuda_ops.gemm(a, b, layout, out=acc, accumulate=True, bn=512)
    torch.testing.assert_close(acc.float(), want + 1.0, rtol=2e-2, atol=2e-2 * float(want.abs().max()))
    cuda_ops.check_status()


@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
def test_cta_pair_gemm_glu_epilogues(act, dev):
    from opentau_b200.ops import cuda_ops, prims
    M, K, I = 1100, 256, 1024
    x = (torch.randn(M, K) * 0.5).to(torch.bfloat16).to(dev)
    w = (torch.randn(2 * I, K) * 0.1).to(torch.bfloat16).to(dev)
    gu, h = cuda_ops.gemm(x, w, "nt", glu=act, bn=512)
    gu1, h1 = cuda_ops.gemm(x, w, "nt", glu=act, bn=256)
    torch.testing.assert_close(gu.float(), gu1.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(h.float(), h1.float(), rtol=1e-2, atol=1e-2)
    cuda_ops.check_status()


@pytest.mark.parametrize("H", [1024, 2048, 2560])
def test_norm_backward_adds_the_residual_gradient_in_the_kernel(H):
    """``rms_bwd`` / ``ada_rms_bwd`` with ``dres``: dx equals the kernel's dx without it plus ``dres`` (bf16), for the
    weighted, the weightless and the adaptive form; the weight / modulation gradients are unchanged."""
    from opentau_b200.ops import cuda_ops
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(H)
    B, S = 3, 37
    x = torch.randn(B, S, H, device=dev, generator=g).to(torch.bfloat16)
    dy = torch.randn(B, S, H, device=dev, generator=g).to(torch.bfloat16)
    dres = torch.randn(B, S, H, device=dev, generator=g).to(torch.bfloat16)
    w = (0.1 * torch.randn(H, device=dev, generator=g)).to(torch.bfloat16)
    mod = (0.1 * torch.randn(B, 3 * H, device=dev, generator=g)).to(torch.bfloat16)
    _, rstd = cuda_ops.rms_fwd(x, w, 1e-6, True)
    for wt in (w, None):
        dx0, dw0 = cuda_ops.rms_bwd(dy, x, wt, rstd, True)
        dx1, dw1 = cuda_ops.rms_bwd(dy, x, wt, rstd, True, dres)
        torch.testing.assert_close(dx1.float(), dx0.float() + dres.float(), rtol=1e-2, atol=2e-2)
        if wt is not None:
            assert torch.equal(dw0, dw1)
    _, rstd_a = cuda_ops.ada_rms_fwd(x, mod, 1e-6)
    a0 = cuda_ops.ada_rms_bwd(dy, x, mod, rstd_a)
    a1 = cuda_ops.ada_rms_bwd(dy, x, mod, rstd_a, dres)
    torch.testing.assert_close(a1[0].float(), a0[0].float() + dres.float(), rtol=1e-2, atol=2e-2)
    assert torch.equal(a0[1], a1[1]) and torch.equal(a0[2], a1[2])
