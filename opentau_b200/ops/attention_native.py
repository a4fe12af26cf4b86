"""ctypes launchers of the block-causal attention kernels: tcgen05 (bf16) and the exact fp32 CUDA-core kernels."""

from __future__ import annotations

import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch
from torch import Tensor

from . import _lib


def _enabled() -> bool:
    return os.environ.get("OPENTAU_B200_DENSE_ATTN", "0") != "1"


def supported(q: Tensor, k: Tensor, v: Tensor) -> bool:
    if not _enabled() or q.dtype != torch.bfloat16:
        return False
    B, Sq, H, D = q.shape
    Hkv = k.shape[2]
    g = H // Hkv
    return D % 8 == 0 and 16 <= D <= 256 and H % Hkv == 0 and g <= 128 and 128 % g == 0


def supported_bwd(q: Tensor, k: Tensor, v: Tensor) -> bool:
    if not supported(q, k, v) or os.environ.get("OPENTAU_B200_DENSE_ATTN_BWD", "0") == "1":
        return False
    g = q.shape[2] // k.shape[2]
    return g <= 32 and 32 % g == 0


def _u8(m: Tensor) -> Tensor:
    """Validity mask as bytes; a bool tensor is reinterpreted (one byte per element, 0 / 1), not converted."""
    m = m.contiguous()
    return m.view(torch.uint8) if m.dtype == torch.bool else m.to(torch.uint8)


def _prep(t: Tensor) -> Tensor:
    if t.stride(3) != 1 or any(s % 8 for s in t.stride()[:3]) or t.data_ptr() % 16:
        t = t.contiguous()
    return t


NUM_SMS = 148


def split_kv(B: int, Sq: int, Sk: int, H: int, Hkv: int, D: int) -> int:
    """Key splits per query tile: only when the tiles alone would leave three quarters of the SMs idle and every split
    still gets two key blocks (a 51-token suffix against a 1000-token prefix: 4 CTAs become 32)."""
    g = H // Hkv
    if D % 4 or g > 128 or 128 % g:
        return 1
    ctas = -(-Sq // (128 // g)) * Hkv * B
    nblk = -(-Sk // (64 if D > 128 else 128))
    if ctas * 4 > NUM_SMS:
        return 1
    return max(1, min(8, NUM_SMS // ctas, nblk // 2))


def attn_fwd(q: Tensor, k: Tensor, v: Tensor, q_blk: Tensor, k_blk: Tensor, q_valid: Tensor, k_valid: Tensor,
             scale: float, nsplit: int | None = None):
    from . import cuda_ops
    B, Sq, H, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    q, k, v = _prep(q), _prep(k), _prep(v)
    o = torch.empty(B, Sq, H * D, dtype=q.dtype, device=q.device)
    lse = torch.empty(B, H, Sq, dtype=torch.float32, device=q.device)
    qb = q_blk.to(torch.int32).contiguous()
    kb = k_blk.to(torch.int32).contiguous()
    qv = _u8(q_valid)
    kv = _u8(k_valid)
    lib = _lib.load("attention_tcgen05")
    args = [c_void_p(q.data_ptr()), c_void_p(k.data_ptr()), c_void_p(v.data_ptr()), c_void_p(o.data_ptr()),
            c_void_p(lse.data_ptr()), c_void_p(qb.data_ptr()), c_void_p(kb.data_ptr()), c_void_p(qv.data_ptr()),
            c_void_p(kv.data_ptr()), c_int(B), c_int(Sq), c_int(Sk), c_int(H), c_int(Hkv), c_int(D),
            c_longlong(q.stride(0)), c_longlong(q.stride(1)), c_longlong(q.stride(2)),
            c_longlong(k.stride(0)), c_longlong(k.stride(1)), c_longlong(k.stride(2)),
            c_longlong(v.stride(0)), c_longlong(v.stride(1)), c_longlong(v.stride(2)), c_float(scale)]
    nsplit = split_kv(B, Sq, Sk, H, Hkv, D) if nsplit is None else nsplit
    if nsplit > 1:
        part_o = torch.empty(nsplit, B, Sq, H, D, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(nsplit, B, H, Sq, 2, dtype=torch.float32, device=q.device)
        rc = lib.otb_attn_fwd_splitkv(*args, c_int(nsplit), c_void_p(part_o.data_ptr()),
                                      c_void_p(part_ml.data_ptr()), c_void_p(cuda_ops.status_pointer()),
                                      cuda_ops._stream())
        cuda_ops.launch_count += 1
    else:
        rc = lib.otb_attn_fwd(*args, c_void_p(cuda_ops.status_pointer()), cuda_ops._stream())
    if rc != 0:
        raise RuntimeError(f"native attn_fwd failed with code {rc} (B={B} Sq={Sq} Sk={Sk} H={H} Hkv={Hkv} D={D})")
    cuda_ops.launch_count += 1
    return o, lse


def attn_bwd(do: Tensor, q: Tensor, k: Tensor, v: Tensor, o: Tensor, lse: Tensor, q_blk: Tensor, k_blk: Tensor,
             q_valid: Tensor, k_valid: Tensor, scale: float):
    """Returns ``(dq, dk, dv)``; ``delta`` scratch and outputs are allocated here."""
    from . import cuda_ops
    B, Sq, H, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    q, k, v = _prep(q), _prep(k), _prep(v)
    o = o.contiguous()
    do = do.contiguous()
    lse = lse.contiguous()
    dq = torch.empty(B, Sq, H, D, dtype=q.dtype, device=q.device)
    dk = torch.empty(B, Sk, Hkv, D, dtype=q.dtype, device=q.device)
    dv = torch.empty(B, Sk, Hkv, D, dtype=q.dtype, device=q.device)
    delta = torch.empty(B, H, Sq, dtype=torch.float32, device=q.device)
    qb = q_blk.to(torch.int32).contiguous()
    kb = k_blk.to(torch.int32).contiguous()
    qv = _u8(q_valid)
    kv = _u8(k_valid)
    rc = _lib.load("attention_bwd_tcgen05").otb_attn_bwd(
        c_void_p(q.data_ptr()), c_void_p(k.data_ptr()), c_void_p(v.data_ptr()), c_void_p(o.data_ptr()),
        c_void_p(do.data_ptr()), c_void_p(lse.data_ptr()), c_void_p(delta.data_ptr()), c_void_p(dq.data_ptr()),
        c_void_p(dk.data_ptr()), c_void_p(dv.data_ptr()), c_void_p(qb.data_ptr()), c_void_p(kb.data_ptr()),
        c_void_p(qv.data_ptr()), c_void_p(kv.data_ptr()), c_int(B), c_int(Sq), c_int(Sk), c_int(H), c_int(Hkv),
        c_int(D), c_longlong(q.stride(0)), c_longlong(q.stride(1)), c_longlong(q.stride(2)),
        c_longlong(k.stride(0)), c_longlong(k.stride(1)), c_longlong(k.stride(2)),
        c_longlong(v.stride(0)), c_longlong(v.stride(1)), c_longlong(v.stride(2)),
        c_float(scale), c_void_p(cuda_ops.status_pointer()), cuda_ops._stream())
    if rc != 0:
        raise RuntimeError(f"native attn_bwd failed with code {rc} (B={B} Sq={Sq} Sk={Sk} H={H} Hkv={Hkv} D={D})")
    cuda_ops.launch_count += 4
    return dq, dk, dv


# ------------------------------------------------------------------------------------------- exact fp32 (CUDA cores)
def supported_f32(q: Tensor, k: Tensor, v: Tensor) -> bool:
    """fp32 CUDA tensors with a head width that is a multiple of 4 up to 256 go to ``csrc/attention_f32.cu``: exact
    fp32 arithmetic without the (B, H, Sq, Sk) score tensor of the dense body."""
    if not _enabled() or q.dtype != torch.float32 or not q.is_cuda:
        return False
    D, H, Hkv = q.shape[3], q.shape[2], k.shape[2]
    return k.dtype == v.dtype == torch.float32 and D % 4 == 0 and 4 <= D <= 256 and H % Hkv == 0


#: score bytes of one 8-sample chunk of the dense evaluation above which the kernels are used whatever the head width
F32_DENSE_SCORE_LIMIT = 1 << 30


def prefer_f32_kernels(q: Tensor, k: Tensor) -> bool:
    """Which fp32 path the dispatcher takes when both can run (``OPENTAU_B200_F32_ATTN=kernel|dense`` forces one).
    Measured on a B200: the kernels need O(S) extra memory instead of the (B, H, Sq, Sk) score tensor and are 2.5 x
    (forward) / 1.1 x (backward) the dense evaluation at head width 64, but at head width 256 the library's fp32 GEMMs
    win (forward 0.9 x, backward 0.3 x) as long as the scores fit.  So: kernels for head widths up to 128, and at any
    width once the scores of a chunk would pass :data:`F32_DENSE_SCORE_LIMIT`."""
    mode = os.environ.get("OPENTAU_B200_F32_ATTN", "auto")
    if mode in ("kernel", "dense"):
        return mode == "kernel"
    B, Sq, H, D = q.shape
    scores = min(B, 8) * H * Sq * k.shape[1] * 4
    return D <= 128 or scores > F32_DENSE_SCORE_LIMIT


def _prep_f32(t: Tensor) -> Tensor:
    if t.stride(3) != 1 or any(s % 4 for s in t.stride()[:3]) or t.data_ptr() % 16:
        t = t.contiguous()
    return t


def _f32_common(q, k, v, q_blk, k_blk, q_valid, k_valid):
    B, Sq, H, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    q, k, v = _prep_f32(q), _prep_f32(k), _prep_f32(v)
    keep = (q, k, v, q_blk.to(torch.int32).contiguous(), k_blk.to(torch.int32).contiguous(), _u8(q_valid), _u8(k_valid))
    dims = [c_int(B), c_int(Sq), c_int(Sk), c_int(H), c_int(Hkv), c_int(D),
            c_longlong(q.stride(0)), c_longlong(q.stride(1)), c_longlong(q.stride(2)),
            c_longlong(k.stride(0)), c_longlong(k.stride(1)), c_longlong(k.stride(2)),
            c_longlong(v.stride(0)), c_longlong(v.stride(1)), c_longlong(v.stride(2))]
    return keep, dims


def attn_f32_fwd(q: Tensor, k: Tensor, v: Tensor, q_blk, k_blk, q_valid, k_valid, scale: float):
    from . import cuda_ops
    B, Sq, H, D = q.shape
    (q, k, v, qb, kb, qv, kv), dims = _f32_common(q, k, v, q_blk, k_blk, q_valid, k_valid)
    o = torch.empty(B, Sq, H * D, dtype=torch.float32, device=q.device)
    lse = torch.empty(B, H, Sq, dtype=torch.float32, device=q.device)
    rc = _lib.load("attention_f32").otb_attn_f32_fwd(
        c_void_p(q.data_ptr()), c_void_p(k.data_ptr()), c_void_p(v.data_ptr()), c_void_p(o.data_ptr()),
        c_void_p(lse.data_ptr()), c_void_p(qb.data_ptr()), c_void_p(kb.data_ptr()), c_void_p(qv.data_ptr()),
        c_void_p(kv.data_ptr()), *dims, c_float(scale), cuda_ops._stream())
    if rc != 0:
        raise RuntimeError(f"fp32 attn_fwd failed with code {rc} (B={B} Sq={Sq} Sk={k.shape[1]} H={H} D={D})")
    cuda_ops.launch_count += 1
    return o, lse


def attn_f32_bwd(do: Tensor, q: Tensor, k: Tensor, v: Tensor, o: Tensor, lse: Tensor, q_blk, k_blk, q_valid, k_valid,
                 scale: float):
    from . import cuda_ops
    B, Sq, H, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    (q, k, v, qb, kb, qv, kv), dims = _f32_common(q, k, v, q_blk, k_blk, q_valid, k_valid)
    o = o.contiguous().float()
    do = do.contiguous().float()
    lse = lse.contiguous()
    dq = torch.empty(B, Sq, H, D, dtype=torch.float32, device=q.device)
    dk = torch.empty(B, Sk, Hkv, D, dtype=torch.float32, device=q.device)
    dv = torch.empty(B, Sk, Hkv, D, dtype=torch.float32, device=q.device)
    delta = torch.empty(B, H, Sq, dtype=torch.float32, device=q.device)
    rc = _lib.load("attention_f32").otb_attn_f32_bwd(
        c_void_p(q.data_ptr()), c_void_p(k.data_ptr()), c_void_p(v.data_ptr()), c_void_p(o.data_ptr()),
        c_void_p(do.data_ptr()), c_void_p(lse.data_ptr()), c_void_p(delta.data_ptr()), c_void_p(dq.data_ptr()),
        c_void_p(dk.data_ptr()), c_void_p(dv.data_ptr()), c_void_p(qb.data_ptr()), c_void_p(kb.data_ptr()),
        c_void_p(qv.data_ptr()), c_void_p(kv.data_ptr()), *dims, c_float(scale), cuda_ops._stream())
    if rc != 0:
        raise RuntimeError(f"fp32 attn_bwd failed with code {rc} (B={B} Sq={Sq} Sk={Sk} H={H} Hkv={Hkv} D={D})")
    cuda_ops.launch_count += 3
    return dq, dk, dv
