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
