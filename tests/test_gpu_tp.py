"""Fused tensor-parallel GEMM kernels on ONE GPU: the ranks are emulated as separate buffers on the same device
and their kernels run one after another.  No launch ever waits for another one: the all-gather GEMM sees ready
flags that are already set, and the GEMM -> reduce-scatter runs its two halves as separate launches (all ranks'
GEMM + peer stores first, then all ranks' reductions, whose counters are complete by then)."""

import ctypes
from ctypes import c_int, c_longlong, c_uint, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
MAXR = 8
BUDGET = 200_000_000


def _arr(tensors):
    return (c_void_p * MAXR)(*[c_void_p(t.data_ptr()) for t in tensors], *[c_void_p(0)] * (MAXR - len(tensors)))


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("world,Ml,N,K,bias", [(2, 256, 512, 256, False), (4, 200, 384, 320, True),
                                                (8, 96, 1024, 128, True), (2, 1100, 4096, 512, False)])
def test_all_gather_gemm_emulated(world, Ml, N, K, bias):
    from opentau_b200.ops import _lib, cuda_ops
    lib = _lib.load("gemm_dist_tcgen05")
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    a = [torch.randn(Ml, K, device=dev).to(torch.bfloat16) for _ in range(world)]
    ws = [(torch.randn(N, K, device=dev) / K ** 0.5).to(torch.bfloat16) for _ in range(world)]
    b = torch.randn(N, device=dev).to(torch.bfloat16) if bias else None
    ready = torch.full((MAXR,), 2, device=dev, dtype=torch.int32)      # every source already published 2 steps
    status = c_void_p(cuda_ops.status_pointer())
    full = torch.cat(a, 0).float()
    nblk = (Ml + 127) // 128
    for r in range(world):
        gathered = torch.zeros(world * Ml, K, device=dev, dtype=torch.bfloat16)
        gcount = torch.zeros(world * nblk + 1, device=dev, dtype=torch.int32)
        for epoch in (1, 2):                                           # the piece counters keep counting
            out = torch.zeros(world * Ml, N, device=dev, dtype=torch.bfloat16)
            rc = lib.otb_ag_gemm_bf16(_arr(a), c_void_p(ws[r].data_ptr()), c_void_p(out.data_ptr()), c_int(Ml),
                                      c_int(N), c_int(K), c_longlong(K), c_longlong(N),
                                      c_void_p(b.data_ptr() if bias else 0), c_void_p(ready.data_ptr()),
                                      c_void_p(gathered.data_ptr()), c_void_p(gcount.data_ptr()), c_int(r),
                                      c_int(world), c_uint(epoch), c_longlong(BUDGET), status, _stream())
            assert rc == 0
            want = full @ ws[r].float().t() + (b.float() if bias else 0)
            torch.testing.assert_close(out.float(), want, atol=3e-2, rtol=2e-2)
        others = [x for i, x in enumerate(a) if i != r]
        got = torch.cat([gathered[i * Ml:(i + 1) * Ml] for i in range(world) if i != r], 0)
        assert torch.equal(got, torch.cat(others, 0))                  # every peer row crossed exactly as is
    cuda_ops.check_status()


@pytest.mark.parametrize("world,Ml,N,Kl,extras", [(2, 256, 512, 256, False), (4, 200, 384, 320, True),
                                                  (8, 96, 1024, 128, True), (2, 700, 4096, 256, False)])
def test_gemm_reduce_scatter_emulated(world, Ml, N, Kl, extras):
    from opentau_b200.ops import _lib, cuda_ops
    lib = _lib.load("gemm_dist_tcgen05")
    dev = torch.device("cuda:0")
    torch.manual_seed(1)
    M = world * Ml
    xs = [torch.randn(M, Kl, device=dev).to(torch.bfloat16) for _ in range(world)]
    ws = [(torch.randn(N, Kl, device=dev) / (Kl * world) ** 0.5).to(torch.bfloat16) for _ in range(world)]
    bias = torch.randn(N, device=dev).to(torch.bfloat16) if extras else None
    res = [torch.randn(Ml, N, device=dev).to(torch.bfloat16) for _ in range(world)] if extras else None
    nblk = (Ml + 127) // 128
    stage = [torch.zeros(world * Ml * N, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    outs = [torch.zeros(Ml, N, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    status = c_void_p(cuda_ops.status_pointer())
    for epoch in (1, 2):                                   # counters keep counting across steps
        counters = counters if epoch == 2 else [torch.zeros(world * nblk, device=dev, dtype=torch.int32)
                                                for _ in range(world)]
        for phase in (1, 2):
            for r in range(world):
                rc = lib.otb_gemm_rs_bf16(
                    c_void_p(xs[r].data_ptr()), c_void_p(ws[r].data_ptr()), c_void_p(outs[r].data_ptr()), c_int(Ml),
                    c_int(N), c_int(Kl), c_longlong(Kl), c_longlong(Kl), c_longlong(N),
                    c_void_p(bias.data_ptr() if extras else 0), c_void_p(res[r].data_ptr() if extras else 0),
                    c_longlong(N), _arr(stage), _arr(counters), c_int(r), c_int(world), c_uint(epoch), c_int(phase),
                    c_longlong(BUDGET), status, _stream())
                assert rc == 0
        cuda_ops.check_status()
        total = sum((x.float() @ w.float().t()).to(torch.bfloat16).float() for x, w in zip(xs, ws))
        for r in range(world):
            want = total[r * Ml:(r + 1) * Ml]
            if extras:
                want = want + bias.float() + res[r].float()
            torch.testing.assert_close(outs[r].float(), want, atol=4e-2, rtol=2e-2)
            assert int(counters[r].min()) == epoch * ((N + (255 if _bn(world, Ml, N) == 256 else 127)) //
                                                      _bn(world, Ml, N))


def _bn(world, Ml, N):
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    m_tiles = world * ((Ml + 127) // 128)
    return 256 if (m_tiles * ((N + 255) // 256) >= sms or N >= 4096) else 128


def test_all_gather_gemm_gives_up_on_a_source_that_never_publishes():
    """A ready flag nobody sets and a ~millisecond budget: the kernel must return with a status, not hang."""
    from opentau_b200.ops import _lib, cuda_ops
    lib = _lib.load("gemm_dist_tcgen05")
    dev = torch.device("cuda:0")
    a = [torch.zeros(128, 64, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    w = torch.zeros(128, 64, device=dev, dtype=torch.bfloat16)
    out = torch.zeros(256, 128, device=dev, dtype=torch.bfloat16)
    ready = torch.zeros(MAXR, device=dev, dtype=torch.int32)
    gathered = torch.zeros(256, 64, device=dev, dtype=torch.bfloat16)
    gcount = torch.zeros(3, device=dev, dtype=torch.int32)
    cuda_ops.check_status()
    rc = lib.otb_ag_gemm_bf16(_arr(a), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), c_int(128), c_int(128),
                              c_int(64), c_longlong(64), c_longlong(128), c_void_p(0), c_void_p(ready.data_ptr()),
                              c_void_p(gathered.data_ptr()), c_void_p(gcount.data_ptr()), c_int(0), c_int(2),
                              c_uint(1), c_longlong(2_000_000), c_void_p(cuda_ops.status_pointer()), _stream())
    assert rc == 0
    with pytest.raises(RuntimeError, match="timed out"):
        cuda_ops.check_status()
    cuda_ops.check_status()          # status was reset; the context is still usable
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0
