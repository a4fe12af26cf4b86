"""Peer-memory step kernels on ONE GPU: the ranks are emulated as separate buffers on the same device and
their kernels run one after another (no kernel ever waits for another launch).  Waits are exercised only
with flags that are already set, or with a flag nobody sets and a tiny budget (the timeout path)."""

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
MAXR = 8


def _table(tensors):
    ptrs = [c_void_p(t.data_ptr()) for t in tensors] + [c_void_p(0)] * (MAXR - len(tensors))
    return (c_void_p * MAXR)(*ptrs)


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def test_fused_step_two_emulated_ranks_matches_reference():
    from opentau_b200.ops import _lib, cuda_ops
    from opentau_b200.ops import reference as ref
    lib = _lib.load("comm_p2p")
    dev = torch.device("cuda:0")
    world, n = 2, 1 << 16
    shard = n // world
    g = [torch.randn(n, device=dev).to(torch.bfloat16) for _ in range(world)]
    p16 = [torch.zeros(n, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    master_full = torch.randn(n, device=dev)
    masters = [master_full[r * shard:(r + 1) * shard].clone() for r in range(world)]
    ms = [torch.zeros(shard, device=dev) for _ in range(world)]
    vs = [torch.zeros(shard, device=dev) for _ in range(world)]
    g32 = [torch.empty(shard, device=dev) for _ in range(world)]
    partial = [torch.zeros(256, device=dev) for _ in range(world)]
    flags = [torch.full((MAXR * 4,), 1, device=dev, dtype=torch.int32) for _ in range(world)]  # epoch 1 already signalled
    norms = [torch.zeros(MAXR, device=dev) for _ in range(world)]
    scale = [torch.zeros(2, device=dev) for _ in range(world)]
    status = c_void_p(cuda_ops.status_pointer())
    for r in range(world):
        rc = lib.otb_comm_reduce_scatter(_table(g), c_int(world), c_longlong(r * shard), c_longlong(shard),
                                         c_void_p(g32[r].data_ptr()), c_void_p(partial[r].data_ptr()), c_int(256),
                                         c_int(2), status, _stream())
        assert rc == 0
    gsum = g[0].float() + g[1].float()
    for r in range(world):
        torch.testing.assert_close(g32[r], gsum[r * shard:(r + 1) * shard])
    for r in (1, 0, 1):   # rank 1 publishes, rank 0 then sees both totals, rank 1 again sees both
        rc = lib.otb_comm_norm_exchange(c_void_p(partial[r].data_ptr()), c_int(256), _table(norms), _table(flags),
                                        c_int(r), c_int(world), c_int(1), c_int(1), c_float(1.0 / world),
                                        c_float(1.0), c_void_p(scale[r].data_ptr()), c_longlong(10_000_000), status,
                                        _stream())
        assert rc == 0
    norm_ref = gsum.pow(2).sum().sqrt().item() / world
    for r in range(world):
        assert abs(scale[r][1].item() - norm_ref) / norm_ref < 1e-4
        assert abs(scale[r][0].item() - min(1.0, 1.0 / (norm_ref + 1e-6)) / world) < 1e-6
    hp = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.01)
    for r in range(world):
        rc = lib.otb_comm_adamw_allgather(c_void_p(masters[r].data_ptr()), c_void_p(g32[r].data_ptr()),
                                          c_void_p(ms[r].data_ptr()), c_void_p(vs[r].data_ptr()), _table(p16),
                                          c_int(world), c_longlong(r * shard), c_longlong(shard), c_float(hp["lr"]),
                                          c_float(hp["beta1"]), c_float(hp["beta2"]), c_float(hp["eps"]),
                                          c_float(hp["wd"]), c_float(1 - hp["beta1"]), c_float(1 - hp["beta2"]),
                                          c_void_p(scale[r].data_ptr()), c_int(64), c_int(2), status, _stream())
        assert rc == 0
    torch.cuda.synchronize()
    cuda_ops.check_status()
    pr, mr, vr = master_full.clone().cpu(), torch.zeros(n), torch.zeros(n)
    ref.adamw_flat(pr, gsum.cpu(), mr, vr, None, lr=hp["lr"], beta1=hp["beta1"], beta2=hp["beta2"], eps=hp["eps"],
                   weight_decay=hp["wd"], step=1, grad_scale=scale[0][0].item())
    assert torch.equal(p16[0], p16[1])          # every "rank" holds the same refreshed parameters
    torch.testing.assert_close(torch.cat(masters).cpu(), pr, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(p16[0].cpu().float(), pr, rtol=1e-2, atol=1e-2)


def test_barrier_wait_times_out_and_reports_status():
    """A flag that nobody sets: the bounded wait must give up, report, and leave the context usable."""
    from opentau_b200.ops import _lib, cuda_ops
    lib = _lib.load("comm_p2p")
    dev = torch.device("cuda:0")
    flags = [torch.zeros(MAXR * 4, device=dev, dtype=torch.int32) for _ in range(2)]
    cuda_ops.check_status()
    status = c_void_p(cuda_ops.status_pointer())
    rc = lib.otb_comm_barrier(_table(flags), c_int(0), c_int(2), c_int(0), c_int(5), c_longlong(2_000_000), status,
                              _stream())
    assert rc == 0
    # while the record stands, the data kernels behind the wait write NOTHING: a late or dead peer can stall a step
    # but cannot get half-written gradients averaged into the weights
    n = 1 << 12
    g = [torch.ones(n, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    g32 = torch.full((n,), 7.0, device=dev)
    partial = torch.full((64,), 7.0, device=dev)
    assert lib.otb_comm_reduce_scatter(_table(g), c_int(2), c_longlong(0), c_longlong(n), c_void_p(g32.data_ptr()),
                                       c_void_p(partial.data_ptr()), c_int(64), c_int(2), status, _stream()) == 0
    p16 = [torch.full((n,), 3.0, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    master, m, v = torch.full((n,), 3.0, device=dev), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    scale = torch.ones(2, device=dev)
    assert lib.otb_comm_adamw_allgather(
        c_void_p(master.data_ptr()), c_void_p(g32.data_ptr()), c_void_p(m.data_ptr()), c_void_p(v.data_ptr()),
        _table(p16), c_int(2), c_longlong(0), c_longlong(n), c_float(0.1), c_float(0.9), c_float(0.95), c_float(1e-8),
        c_float(0.0), c_float(0.1), c_float(0.05), c_void_p(scale.data_ptr()), c_int(16), c_int(2), status,
        _stream()) == 0
    torch.cuda.synchronize()
    assert float(g32.min()) == 7.0 and float(partial.min()) == 7.0 and float(master.min()) == 3.0
    assert float(p16[1].float().min()) == 3.0 and float(m.abs().max()) == 0.0
    with pytest.raises(RuntimeError, match="timed out"):
        cuda_ops.check_status()
    cuda_ops.check_status()                       # status word was reset
    x = torch.ones(8, device=dev)
    assert x.sum().item() == 8.0                  # the context still works
    assert flags[1][0].item() == 5                # our own signal was delivered before the wait
