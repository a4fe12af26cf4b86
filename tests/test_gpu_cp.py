"""Context-parallel attention kernel on ONE GPU: the ranks are emulated as separate K/V shards on the same device and
each rank's kernel runs alone (ready flags already set), so no launch waits for another one.  The result must equal
the single-GPU kernel on the full sequence."""

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
MAXR = 8
BUDGET = 400_000_000


def _arr(tensors):
    return (c_void_p * MAXR)(*[c_void_p(t.data_ptr()) for t in tensors], *[c_void_p(0)] * (MAXR - len(tensors)))


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _run_rank(lib, r, W, q, ks, vs, q_blk, k_blk_all, q_valid, k_valid_all, scale, ready, state, epoch, budget=BUDGET,
              copiers=4):
    from opentau_b200.ops import cuda_ops
    B, Sl, H, D = q.shape
    Hkv = ks[0].shape[2]
    o = torch.zeros(B, Sl, H, D, device=q.device, dtype=torch.bfloat16)
    lse = torch.zeros(B, H, Sl, device=q.device)
    rc = lib.otb_attn_fwd_cp(
        c_void_p(q.data_ptr()), c_void_p(o.data_ptr()), c_void_p(lse.data_ptr()), c_void_p(q_blk.data_ptr()),
        c_void_p(k_blk_all.data_ptr()), c_void_p(q_valid.data_ptr()), c_void_p(k_valid_all.data_ptr()), c_int(B),
        c_int(Sl), c_int(Sl), c_int(H), c_int(Hkv), c_int(D), c_longlong(q.stride(0)), c_longlong(q.stride(1)),
        c_longlong(q.stride(2)), _arr(ks), _arr(vs), c_void_p(state["kg"].data_ptr()), c_void_p(state["vg"].data_ptr()),
        c_void_p(state["gcount"].data_ptr()), c_void_p(ready.data_ptr()), c_int(r), c_int(W), c_uint(epoch),
        c_int(copiers), c_float(scale), c_longlong(budget), c_void_p(cuda_ops.status_pointer()), _stream())
    assert rc == 0
    return o.view(B, Sl, H * D), lse


@pytest.mark.parametrize("W,B,Sl,H,Hkv,D", [(2, 2, 256, 8, 1, 256), (4, 1, 200, 8, 4, 128), (8, 2, 96, 4, 4, 64),
                                             (2, 1, 1100, 8, 2, 256)])
def test_cp_attention_emulated_matches_single_gpu_kernel(W, B, Sl, H, Hkv, D):
    from opentau_b200.ops import _lib, cuda_ops, prims
    lib = _lib.load("attention_cp_tcgen05")
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    S = W * Sl
    q = torch.randn(B, S, H, D, device=dev).to(torch.bfloat16)
    k = torch.randn(B, S, Hkv, D, device=dev).to(torch.bfloat16)
    v = torch.randn(B, S, Hkv, D, device=dev).to(torch.bfloat16)
    blk = (torch.arange(S, device=dev, dtype=torch.int32) // 75)[None].expand(B, S).contiguous()
    valid = torch.rand(B, S, device=dev) > 0.05
    scale = D ** -0.5
    want_o, want_lse = prims.attn_fwd(q, k, v, blk, blk, valid, valid, scale)
    ks = [k[:, r * Sl:(r + 1) * Sl].contiguous() for r in range(W)]
    vs = [v[:, r * Sl:(r + 1) * Sl].contiguous() for r in range(W)]
    ready = torch.full((MAXR,), 2, device=dev, dtype=torch.int32)
    bn = int(lib.otb_attn_cp_block(c_int(D)))
    vu8 = valid.to(torch.uint8).contiguous()
    for r in range(W):
        state = {"kg": torch.zeros(W * B * Sl * Hkv * D, device=dev, dtype=torch.bfloat16),
                 "vg": torch.zeros(W * B * Sl * Hkv * D, device=dev, dtype=torch.bfloat16),
                 "gcount": torch.zeros(W * B * ((Sl + bn - 1) // bn + 1) + 1, device=dev, dtype=torch.int32)}
        qr = q[:, r * Sl:(r + 1) * Sl].contiguous()
        for epoch in (1, 2):                                   # the piece counters keep counting across steps
            o, lse = _run_rank(lib, r, W, qr, ks, vs, blk[:, r * Sl:(r + 1) * Sl].contiguous(), blk,
                               vu8[:, r * Sl:(r + 1) * Sl].contiguous(), vu8, scale, ready, state, epoch)
            torch.testing.assert_close(o.float(), want_o[:, r * Sl:(r + 1) * Sl].float(), atol=2e-2, rtol=2e-2)
            torch.testing.assert_close(lse, want_lse[:, :, r * Sl:(r + 1) * Sl], atol=2e-3, rtol=1e-3)
        # the gathered buffers hold every OTHER rank's shard exactly (the own shard is read in place)
        kg = state["kg"].view(W, B, Sl, Hkv, D)
        assert all(torch.equal(kg[s], ks[s]) for s in range(W) if s != r)
    cuda_ops.check_status()


def test_cp_attention_gives_up_when_a_peer_never_publishes():
    from opentau_b200.ops import _lib, cuda_ops
    lib = _lib.load("attention_cp_tcgen05")
    dev = torch.device("cuda:0")
    B, Sl, H, Hkv, D, W = 1, 128, 4, 4, 64, 2
    q = torch.zeros(B, Sl, H, D, device=dev, dtype=torch.bfloat16)
    ks = [torch.zeros(B, Sl, Hkv, D, device=dev, dtype=torch.bfloat16) for _ in range(W)]
    blk_all = torch.zeros(B, W * Sl, device=dev, dtype=torch.int32)
    ok_all = torch.ones(B, W * Sl, device=dev, dtype=torch.uint8)
    ready = torch.zeros(MAXR, device=dev, dtype=torch.int32)          # rank 1 never publishes
    state = {"kg": torch.zeros(W * B * Sl * Hkv * D, device=dev, dtype=torch.bfloat16),
             "vg": torch.zeros(W * B * Sl * Hkv * D, device=dev, dtype=torch.bfloat16),
             "gcount": torch.zeros(W * B * 2 + 1, device=dev, dtype=torch.int32)}
    cuda_ops.check_status()
    _run_rank(lib, 0, W, q, ks, ks, blk_all[:, :Sl].contiguous(), blk_all, ok_all[:, :Sl].contiguous(), ok_all, 0.125,
              ready, state, 1, budget=2_000_000)
    with pytest.raises(RuntimeError, match="timed out"):
        cuda_ops.check_status()
    cuda_ops.check_status()
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0
