"""Block-causal attention launchers for CUDA tensors.

bf16 tensors go to the tcgen05 kernels (``csrc/attention_tcgen05.cu``, ``csrc/attention_bwd_tcgen05.cu``), fp32
tensors to the exact CUDA-core kernels (``csrc/attention_f32.cu``); geometries neither takes (and
``OPENTAU_B200_DENSE_ATTN=1``) use a dense PyTorch body evaluated in batch chunks.
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import reference as ref


def _dense_fwd_chunk(q, k, v, mask, scale):
    B, Sq, H, D = q.shape
    Hkv = k.shape[2]
    g = H // Hkv
    s = torch.einsum("bqhgd,bkhd->bhgqk", q.view(B, Sq, Hkv, g, D), k).float() * scale
    s = s.masked_fill(~mask[:, None, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    any_vis = mask.any(-1)[:, None, None, :]
    lse = torch.where(any_vis, lse, torch.zeros_like(lse))
    p = torch.exp(s - lse[..., None])
    p = torch.where(any_vis[..., None], p, torch.zeros_like(p)).to(v.dtype)
    o = torch.einsum("bhgqk,bkhd->bqhgd", p, v)
    return o.reshape(B, Sq, H * D), lse.reshape(B, H, Sq)


def dense_attn_fwd(q, k, v, q_blk, k_blk, q_valid, k_valid, scale, chunk: int = 8):
    B = q.shape[0]
    outs, lses = [], []
    for b0 in range(0, B, chunk):
        sl = slice(b0, min(B, b0 + chunk))
        mask = ref.dense_mask_from_blocks(q_blk[sl], k_blk[sl], q_valid[sl], k_valid[sl])
        o, l = _dense_fwd_chunk(q[sl], k[sl], v[sl], mask, scale)
        outs.append(o), lses.append(l)
    return torch.cat(outs), torch.cat(lses)


def dense_attn_bwd(do, q, k, v, o, lse, q_blk, k_blk, q_valid, k_valid, scale, chunk: int = 8):
    B, Sq, H, D = q.shape
    Hkv = k.shape[2]
    g = H // Hkv
    dq = torch.empty(B, Sq, H, D, dtype=q.dtype, device=q.device)
    dk = torch.empty(B, k.shape[1], Hkv, D, dtype=k.dtype, device=q.device)
    dv = torch.empty_like(dk)
    for b0 in range(0, B, chunk):
        sl = slice(b0, min(B, b0 + chunk))
        n = sl.stop - sl.start
        mask = ref.dense_mask_from_blocks(q_blk[sl], k_blk[sl], q_valid[sl], k_valid[sl])
        qc = q[sl].view(n, Sq, Hkv, g, D)
        s = torch.einsum("bqhgd,bkhd->bhgqk", qc, k[sl]).float() * scale
        p = torch.exp(s - lse[sl].view(n, Hkv, g, Sq)[..., None])
        p = torch.where(mask[:, None, None], p, torch.zeros_like(p))
        doc = do[sl].view(n, Sq, Hkv, g, D)
        delta = (doc.float() * o[sl].view(n, Sq, Hkv, g, D).float()).sum(-1).permute(0, 2, 3, 1)
        pb = p.to(v.dtype)
        dv[sl] = torch.einsum("bhgqk,bqhgd->bkhd", pb, doc)
        dp = torch.einsum("bqhgd,bkhd->bhgqk", doc, v[sl]).float()
        ds = (p * (dp - delta[..., None]) * scale).to(q.dtype)
        dq[sl] = torch.einsum("bhgqk,bkhd->bqhgd", ds, k[sl]).reshape(n, Sq, H, D)
        dk[sl] = torch.einsum("bhgqk,bqhgd->bkhd", ds, qc)
    return dq, dk, dv


def attn_fwd(q: Tensor, k: Tensor, v: Tensor, q_blk, k_blk, q_valid, k_valid, scale: float):
    from . import attention_native
    if attention_native.supported(q, k, v):
        return attention_native.attn_fwd(q, k, v, q_blk, k_blk, q_valid, k_valid, scale)
    if attention_native.supported_f32(q, k, v) and attention_native.prefer_f32_kernels(q, k):
        return attention_native.attn_f32_fwd(q, k, v, q_blk, k_blk, q_valid, k_valid, scale)
    return dense_attn_fwd(q, k, v, q_blk, k_blk, q_valid, k_valid, scale)


def attn_bwd(do, q, k, v, o, lse, q_blk, k_blk, q_valid, k_valid, scale):
    from . import attention_native
    if attention_native.supported_bwd(q, k, v):
        return attention_native.attn_bwd(do, q, k, v, o, lse, q_blk, k_blk, q_valid, k_valid, scale)
    if attention_native.supported_f32(q, k, v) and attention_native.prefer_f32_kernels(q, k):
        return attention_native.attn_f32_bwd(do, q, k, v, o, lse, q_blk, k_blk, q_valid, k_valid, scale)
    return dense_attn_bwd(do, q, k, v, o, lse, q_blk, k_blk, q_valid, k_valid, scale)
