"""Tiny pi0.5 on the GPU through the native kernels: parity with the CPU oracle, training step, sampler
replayed from a CUDA graph."""

import pytest
import torch

from helpers import tiny_batch, tiny_pi05

pytestmark = pytest.mark.gpu


def _pair(seed=0):
    cpu = tiny_pi05(seed=seed)
    gpu = tiny_pi05(seed=seed)
    gpu.load_state_dict(cpu.state_dict())
    return cpu, gpu.to("cuda").to(torch.bfloat16)


def test_loss_parity_with_cpu_fp32_oracle():
    from opentau_b200.ops import cuda_ops
    cpu, gpu = _pair()
    for n, p in cpu.named_parameters():        # open the adaptive-norm gates so the expert path matters
        if ".dense." in n:
            torch.nn.init.normal_(p, std=0.05)
    gpu.load_state_dict(cpu.state_dict())
    gpu = gpu.to("cuda").to(torch.bfloat16)
    b = tiny_batch()
    noise, time = torch.randn(4, 10, 32), torch.full((4,), 0.4)
    ref = cpu(b, noise=noise, time=time)
    bg = {k: v.cuda() for k, v in b.items()}
    out = gpu(bg, noise=noise.cuda(), time=time.cuda())
    cuda_ops.check_status()
    assert abs(out["MSE"].item() - ref["MSE"].item()) / ref["MSE"].item() < 3e-2
    assert abs(out["CE"].item() - ref["CE"].item()) / ref["CE"].item() < 3e-2
    (out["MSE"] + out["CE"]).backward()
    (ref["MSE"] + ref["CE"]).backward()
    cuda_ops.check_status()
    checked = 0
    for (n, pc), (_, pg) in zip(cpu.named_parameters(), gpu.named_parameters()):
        if pc.grad is None or pc.grad.abs().max() < 1e-6 or pc.numel() < 512:
            continue
        a, c = pg.grad.float().cpu().flatten(), pc.grad.flatten()
        cos = torch.nn.functional.cosine_similarity(a, c, dim=0).item()
        assert cos > 0.98, f"{n}: cosine {cos}"
        checked += 1
    assert checked > 10


def test_training_reduces_loss_on_gpu():
    from opentau_b200.ops import cuda_ops
    from opentau_b200.parallel.engine import OptimHyper, TrainEngine
    pol = tiny_pi05(seed=1).to(torch.bfloat16).train()
    eng = TrainEngine(pol, OptimHyper(lr=2e-3, grad_clip_norm=1.0), device="cuda")
    b = tiny_batch(device="cuda")
    noise, time = torch.randn(4, 10, 32, device="cuda"), torch.full((4,), 0.5, device="cuda")
    first = last = None
    for _ in range(12):
        out = pol(b, noise=noise, time=time)
        loss = out["MSE"] + out["CE"]
        loss.backward()
        eng.optimizer_step()
        first = loss.item() if first is None else first
        last = loss.item()
    cuda_ops.check_status()
    assert last < 0.8 * first


def test_cuda_graph_sampler_matches_eager():
    from opentau_b200.ops import cuda_ops
    pol = tiny_pi05(seed=2).to("cuda").to(torch.bfloat16).eval()
    b = tiny_batch(device="cuda")
    noise = torch.randn(4, 10, 32, device="cuda")
    eager = pol.sample_actions(b, noise=noise)
    pol.enable_cuda_graphs(True)
    g1 = pol.sample_actions(b, noise=noise)
    g2 = pol.sample_actions(b, noise=noise)           # replay
    other = pol.sample_actions(b, noise=noise * 0.5)  # replay with new inputs
    cuda_ops.check_status()
    torch.testing.assert_close(g1, eager, rtol=1e-3, atol=1e-3)
    assert torch.equal(g1, g2)
    assert not torch.allclose(other, g1)
    assert pol._graph_runner.num_graphs == 1
