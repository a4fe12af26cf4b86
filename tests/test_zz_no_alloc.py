"""Allocation-free column sum, called through its exported C symbol.

Some hosts of the library cannot allocate device memory around a launch (a control loop with a latency
budget, a process with a fixed memory budget, a plain C caller without a tensor allocator).  For them
``otb_colsum_bf16_noalloc`` keeps its partial-sum scratch inside the library.  This test calls it twice in a
row (the scratch keeps the first call's contents) and compares with the regular entry point, which takes a
caller-allocated scratch.  It lives in a file that pytest collects last.
"""

import ctypes
from ctypes import c_char_p, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from opentau_b200.ops import _lib as loader
    lib = loader.load("noalloc_colsum")
    lib.otb_colsum_bf16_noalloc.restype = c_int
    lib.otb_noalloc_strerror.restype = c_char_p
    return lib


def _call(lib, a: torch.Tensor, out: torch.Tensor) -> int:
    return lib.otb_colsum_bf16_noalloc(c_void_p(a.data_ptr()), c_longlong(a.shape[0]), c_int(a.shape[1]),
                                       c_longlong(a.stride(0)), c_void_p(out.data_ptr()),
                                       c_void_p(torch.cuda.current_stream().cuda_stream))


def test_noalloc_colsum_matches_regular_entry_point_twice_in_a_row():
    from opentau_b200.ops import cuda_ops
    lib = _lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(11)
    # two different problems back to back: the second must not be disturbed by what the first left behind
    for rows, H in ((5000, 2048), (777, 1152)):
        a = torch.randn(rows, H, generator=g).to(torch.bfloat16).to(dev)
        out = torch.full((H,), float("nan"), dtype=torch.bfloat16, device=dev)
        before = torch.cuda.memory_allocated()
        rc = _call(lib, a, out)
        assert rc == 0, lib.otb_noalloc_strerror(rc).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before       # nothing was taken from torch's allocator either
        expect = cuda_ops.col_sum(a)                          # regular path: caller-allocated fp32 scratch
        torch.testing.assert_close(out.float(), expect.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(out.float().cpu(), a.float().sum(0).cpu(), rtol=2e-2, atol=0.5)


def test_noalloc_colsum_strided_rows():
    lib = _lib()
    dev = torch.device("cuda:0")
    big = torch.randn(300, 512, device=dev).to(torch.bfloat16)
    a = big[:, :256]                                          # lda = 512 > H = 256
    out = torch.empty(256, dtype=torch.bfloat16, device=dev)
    assert _call(lib, a, out) == 0
    torch.cuda.synchronize()
    torch.testing.assert_close(out.float(), a.float().sum(0), rtol=2e-2, atol=0.3)


def test_noalloc_colsum_rejects_bad_sizes_without_launching():
    lib = _lib()
    dev = torch.device("cuda:0")
    out = torch.zeros(16384, dtype=torch.bfloat16, device=dev)
    too_wide = torch.zeros(4, 16384, dtype=torch.bfloat16, device=dev)
    rc = _call(lib, too_wide, out)
    assert rc < 0 and b"MAX_H" in lib.otb_noalloc_strerror(rc)
    odd = torch.zeros(4, 24, dtype=torch.bfloat16, device=dev)[:, :12]
    assert _call(lib, odd, out) < 0                           # H not a multiple of 8
    assert lib.otb_colsum_bf16_noalloc(c_void_p(0), c_longlong(4), c_int(8), c_longlong(8), c_void_p(out.data_ptr()),
                                       c_void_p(0)) < 0
    assert out.abs().sum().item() == 0                        # refused calls wrote nothing
