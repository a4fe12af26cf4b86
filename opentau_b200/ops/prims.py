"""Non-differentiable primitives: each is one kernel launch on a B200, one torch call on CPU.

The autograd functions in ``fused.py`` are composed from these, so the same backward code is
exercised on CPU (against plain autograd of ``reference.py``) and on the GPU (kernels).
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import Tensor

from . import oracle_mode
from . import reference as ref

GLU_BLOCK = 32  # gate/up rows of a fused gate_up weight alternate in blocks of this many


def _cuda(x: Tensor) -> bool:
    return x.is_cuda and not oracle_mode() and x.dtype == torch.bfloat16


# ----------------------------------------------------------------------------- GEMMs
def mm_nt(a: Tensor, b: Tensor, bias: Tensor | None = None, residual: Tensor | None = None,
          out: Tensor | None = None, accumulate: bool = False, out_dtype: torch.dtype | None = None) -> Tensor:
    """``a (M,K) @ b (N,K).T`` (+bias over N) (+residual (M,N)); fp32 accumulate."""
    if _cuda(a):
        from . import cuda_ops
        return cuda_ops.gemm(a, b, "nt", bias=bias, residual=residual, out=out, accumulate=accumulate,
                             out_dtype=out_dtype)
    y = a @ b.t()
    if bias is not None:
        y = y + bias
    if residual is not None:
        y = y + residual
    if out_dtype is not None:
        y = y.to(out_dtype)
    if out is not None:
        if accumulate:
            out.add_(y)
        else:
            out.copy_(y)
        return out
    return y


def mm_nn(a: Tensor, b: Tensor, out: Tensor | None = None, accumulate: bool = False,
          residual: Tensor | None = None) -> Tensor:
    """``a (M,K) @ b (K,N)``."""
    if _cuda(a):
        from . import cuda_ops
        return cuda_ops.gemm(a, b, "nn", residual=residual, out=out, accumulate=accumulate)
    y = a @ b
    if residual is not None:
        y = y + residual
    if out is not None:
        if accumulate:
            out.add_(y)
        else:
            out.copy_(y)
        return out
    return y


def mm_tn(a: Tensor, b: Tensor, out: Tensor | None = None, accumulate: bool = False) -> Tensor:
    """``a (K,M).T @ b (K,N)`` -> ``(M,N)``; the weight-gradient shape."""
    if _cuda(a):
        from . import cuda_ops
        return cuda_ops.gemm(a, b, "tn", out=out, accumulate=accumulate)
    y = a.t() @ b
    if out is not None:
        if accumulate:
            out.add_(y.to(out.dtype))
        else:
            out.copy_(y)
        return out
    return y


def col_sum(a: Tensor) -> Tensor:
    """Sum over rows of ``(M,N)`` in fp32 (bias gradient)."""
    if _cuda(a):
        from . import cuda_ops
        return cuda_ops.col_sum(a)
    return a.float().sum(0).to(a.dtype)


def mm_nt_glu(x: Tensor, w_gu: Tensor, act: str, keep_gu: bool = True) -> tuple[Tensor | None, Tensor]:
    """``gu = x @ w_gu.T`` and ``h = act(gate) * up`` in one launch (activation in the GEMM epilogue)."""
    if _cuda(x):
        from . import cuda_ops
        res = cuda_ops.gemm(x, w_gu, "nt", glu=act, store_out=keep_gu)
        return res if keep_gu else (None, res)
    gu = x @ w_gu.t()
    return (gu if keep_gu else None), glu_fwd(gu, act)


# ----------------------------------------------------------------------------- norms
def rms_fwd(x: Tensor, w: Tensor | None, eps: float, unit_offset: bool) -> tuple[Tensor, Tensor]:
    """Returns ``(y, rstd)``; ``x (..., H)`` flattened to rows, rstd fp32 ``(rows,)``."""
    if _cuda(x):
        from . import cuda_ops
        return cuda_ops.rms_fwd(x, w, eps, unit_offset)
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
    y = xf * rstd[..., None]
    if w is not None:
        y = y * ((1.0 + w.float()) if unit_offset else w.float())
    return y.to(x.dtype), rstd.reshape(-1)


def rms_bwd(dy: Tensor, x: Tensor, w: Tensor | None, rstd: Tensor, unit_offset: bool,
            dres: Tensor | None = None) -> tuple[Tensor, Tensor | None]:
    """``dres``: the gradient that reached ``x`` through a residual branch; it is added to ``dx`` (inside the kernel on
    the GPU)."""
    if _cuda(x):
        from . import cuda_ops
        if dres is not None and dres.dtype != x.dtype:
            dres = dres.to(x.dtype)
        return cuda_ops.rms_bwd(dy, x, w, rstd, unit_offset, dres)
    H = x.shape[-1]
    xf = x.float().reshape(-1, H)
    dyf = dy.float().reshape(-1, H)
    xhat = xf * rstd[:, None]
    if w is not None:
        wf = (1.0 + w.float()) if unit_offset else w.float()
        dw = (dyf * xhat).sum(0).to(w.dtype)
        g = dyf * wf
    else:
        dw = None
        g = dyf
    dx = (g - xhat * (g * xhat).mean(-1, keepdim=True)) * rstd[:, None]
    if dres is not None:
        dx = dx + dres.float().reshape(-1, H)
    return dx.reshape(x.shape).to(x.dtype), dw


def ada_rms_fwd(x: Tensor, mod: Tensor, eps: float) -> tuple[Tensor, Tensor]:
    """``x (B,S,H)``, ``mod (B,3H)|(B,S,3H)`` -> ``(y, rstd)``; gate is a view of ``mod``."""
    if _cuda(x):
        from . import cuda_ops
        return cuda_ops.ada_rms_fwd(x, mod, eps)
    y, _ = ref.ada_rms_norm(x, mod, eps)
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + eps).reshape(-1)
    return y, rstd


def ada_rms_bwd(dy: Tensor, x: Tensor, mod: Tensor, rstd: Tensor,
                dres: Tensor | None = None) -> tuple[Tensor, Tensor, Tensor]:
    """Returns ``(dx, dscale, dshift)`` with dscale/dshift shaped like the matching ``mod`` chunk; ``dres`` as in
    :func:`rms_bwd`."""
    if _cuda(x):
        from . import cuda_ops
        if dres is not None and dres.dtype != x.dtype:
            dres = dres.to(x.dtype)
        return cuda_ops.ada_rms_bwd(dy, x, mod, rstd, dres)
    B, S, H = x.shape
    m = mod if mod.dim() == 3 else mod[:, None, :]
    scale = m[..., :H].float()
    xf, dyf = x.float(), dy.float()
    xhat = xf * rstd.view(B, S, 1)
    g = dyf * (1.0 + scale)
    dx = (g - xhat * (g * xhat).mean(-1, keepdim=True)) * rstd.view(B, S, 1)
    if dres is not None:
        dx = dx + dres.float()
    dscale = dyf * xhat
    dshift = dyf
    if mod.dim() == 2:
        dscale, dshift = dscale.sum(1), dshift.sum(1)
    return dx.to(x.dtype), dscale.to(mod.dtype), dshift.to(mod.dtype)


def ln_fwd(x: Tensor, w: Tensor, b: Tensor, eps: float) -> tuple[Tensor, Tensor, Tensor]:
    if _cuda(x):
        from . import cuda_ops
        return cuda_ops.ln_fwd(x, w, b, eps)
    xf = x.float()
    mean = xf.mean(-1)
    rstd = torch.rsqrt(xf.var(-1, unbiased=False) + eps)
    y = (xf - mean[..., None]) * rstd[..., None] * w.float() + b.float()
    return y.to(x.dtype), mean.reshape(-1), rstd.reshape(-1)


def ln_bwd(dy: Tensor, x: Tensor, w: Tensor, mean: Tensor, rstd: Tensor):
    if _cuda(x) and x.dtype == torch.bfloat16 and dy.dtype == torch.bfloat16:
        from . import cuda_ops
        return cuda_ops.ln_bwd(dy, x, w, mean, rstd)
    H = x.shape[-1]
    xf = x.float().reshape(-1, H)
    dyf = dy.float().reshape(-1, H)
    xhat = (xf - mean[:, None]) * rstd[:, None]
    dw = (dyf * xhat).sum(0).to(w.dtype)
    db = dyf.sum(0).to(w.dtype)
    g = dyf * w.float()
    dx = (g - g.mean(-1, keepdim=True) - xhat * (g * xhat).mean(-1, keepdim=True)) * rstd[:, None]
    return dx.reshape(x.shape).to(x.dtype), dw, db


# ----------------------------------------------------------------------------- GLU
def _split_glu(gu: Tensor) -> tuple[Tensor, Tensor]:
    v = gu.unflatten(-1, (-1, 2, GLU_BLOCK))
    return v[..., 0, :], v[..., 1, :]


def glu_fwd(gu: Tensor, act: str) -> Tensor:
    """``act(gate) * up`` for a block-interleaved ``[g32|u32|g32|u32…]`` last dim."""
    if _cuda(gu):
        from . import cuda_ops
        return cuda_ops.glu_fwd(gu, act)
    g, u = _split_glu(gu)
    gf = g.float()
    a = F.gelu(gf, approximate="tanh") if act == "gelu_tanh" else F.silu(gf)
    return (a * u.float()).flatten(-2).to(gu.dtype)


def glu_bwd(gu: Tensor, dh: Tensor, act: str, inplace: bool = False) -> Tensor:
    """Gradient w.r.t. the interleaved ``gu``; may overwrite ``gu`` when ``inplace``."""
    if _cuda(gu):
        from . import cuda_ops
        return cuda_ops.glu_bwd(gu, dh, act, inplace)
    g, u = _split_glu(gu)
    gf, uf = g.float(), u.float()
    dhf = dh.float().unflatten(-1, (-1, GLU_BLOCK))
    if act == "gelu_tanh":
        c = math.sqrt(2.0 / math.pi)
        inner = c * (gf + 0.044715 * gf**3)
        t = torch.tanh(inner)
        a = 0.5 * gf * (1 + t)
        da = 0.5 * (1 + t) + 0.5 * gf * (1 - t * t) * c * (1 + 3 * 0.044715 * gf * gf)
    else:
        s = torch.sigmoid(gf)
        a = gf * s
        da = s * (1 + gf * (1 - s))
    dg = dhf * uf * da
    du = dhf * a
    return torch.stack([dg, du], dim=-2).flatten(-3).to(gu.dtype)


def interleave_gate_up(gate_w: Tensor, up_w: Tensor) -> Tensor:
    """Rows of the fused weight: 32 gate rows, 32 up rows, 32 gate rows, …"""
    I, K = gate_w.shape
    return torch.stack([gate_w.view(I // GLU_BLOCK, GLU_BLOCK, K), up_w.view(I // GLU_BLOCK, GLU_BLOCK, K)],
                       dim=1).reshape(2 * I, K)


def deinterleave_gate_up(w: Tensor) -> tuple[Tensor, Tensor]:
    I2, K = w.shape
    v = w.view(I2 // (2 * GLU_BLOCK), 2, GLU_BLOCK, K)
    return v[:, 0].reshape(I2 // 2, K), v[:, 1].reshape(I2 // 2, K)


# ----------------------------------------------------------------------------- rotary
def rope_fwd(x: Tensor, cos: Tensor, sin: Tensor, inverse: bool = False) -> Tensor:
    """Rotate ``x (B,S,H,D)`` (any strides on B,S,H) -> contiguous result; ``inverse`` rotates
    by the negative angle (the backward)."""
    if _cuda(x):
        from . import cuda_ops
        return cuda_ops.rope_fwd(x, cos, sin, inverse)
    return ref.apply_rope(x, cos, -sin if inverse else sin)


# ----------------------------------------------------------------------------- attention
def attn_fwd(q, k, v, q_blk, k_blk, q_valid, k_valid, scale) -> tuple[Tensor, Tensor]:
    """Returns ``(o (B,Sq,H*D), lse (B,H,Sq) fp32)``; rows that see no key give o=0, lse=0."""
    if _cuda(q):
        from . import cuda_ops
        return cuda_ops.attn_fwd(q, k, v, q_blk, k_blk, q_valid, k_valid, scale)
    B, Sq, H, D = q.shape
    Hkv = k.shape[2]
    g = H // Hkv
    mask = ref.dense_mask_from_blocks(q_blk, k_blk, q_valid, k_valid)
    s = torch.einsum("bqhgd,bkhd->bhgqk", q.float().view(B, Sq, Hkv, g, D), k.float()) * scale
    s = s.masked_fill(~mask[:, None, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    any_vis = mask.any(-1)[:, None, None, :]
    lse = torch.where(any_vis, lse, torch.zeros_like(lse))
    p = torch.exp(s - lse[..., None])
    p = torch.where(any_vis[..., None], p, torch.zeros_like(p))
    o = torch.einsum("bhgqk,bkhd->bqhgd", p.to(v.dtype).float(), v.float())
    return o.reshape(B, Sq, H * D).to(q.dtype), lse.reshape(B, H, Sq)


def attn_bwd(do, q, k, v, o, lse, q_blk, k_blk, q_valid, k_valid, scale):
    """Returns ``(dq, dk, dv)`` shaped like q, k, v (dk/dv summed over the GQA group)."""
    if _cuda(q):
        from . import cuda_ops
        return cuda_ops.attn_bwd(do, q, k, v, o, lse, q_blk, k_blk, q_valid, k_valid, scale)
    B, Sq, H, D = q.shape
    Hkv = k.shape[2]
    g = H // Hkv
    mask = ref.dense_mask_from_blocks(q_blk, k_blk, q_valid, k_valid)
    qf = q.float().view(B, Sq, Hkv, g, D)
    kf, vf = k.float(), v.float()
    s = torch.einsum("bqhgd,bkhd->bhgqk", qf, kf) * scale
    p = torch.exp(s - lse.view(B, Hkv, g, Sq)[..., None])
    p = torch.where(mask[:, None, None], p, torch.zeros_like(p))
    dof = do.float().view(B, Sq, Hkv, g, D)
    of = o.float().view(B, Sq, Hkv, g, D)
    delta = (dof * of).sum(-1).permute(0, 2, 3, 1)  # (B,Hkv,g,Sq)
    dv = torch.einsum("bhgqk,bqhgd->bkhd", p, dof)
    dp = torch.einsum("bqhgd,bkhd->bhgqk", dof, vf)
    ds = p * (dp - delta[..., None]) * scale
    dq = torch.einsum("bhgqk,bkhd->bqhgd", ds, kf).reshape(B, Sq, H, D)
    dk = torch.einsum("bhgqk,bqhgd->bkhd", ds, qf)
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


# ----------------------------------------------------------------------------- CE
def linear_ce_fwd(h: Tensor, w: Tensor, bias: Tensor | None, labels: Tensor) -> tuple[Tensor, Tensor]:
    """Per-row CE of ``h @ w.T + b`` and the fp32 logsumexp (saved for backward)."""
    if _cuda(h):
        from . import cuda_ops
        return cuda_ops.linear_ce_fwd(h, w, bias, labels)
    logits = F.linear(h, w, bias).float()
    lse = torch.logsumexp(logits, dim=-1)
    tgt = logits.gather(1, labels[:, None]).squeeze(1)
    return lse - tgt, lse


def linear_ce_bwd(dloss: Tensor, h: Tensor, w: Tensor, bias: Tensor | None, labels: Tensor, lse: Tensor,
                  dw_into: Tensor | None = None):
    """Returns ``(dh, dw, dbias)`` for per-row upstream gradients ``dloss (N,)``; with ``dw_into`` the weight
    gradient is accumulated into that buffer and ``dw`` is None."""
    if _cuda(h):
        from . import cuda_ops
        if dw_into is not None and (dw_into.dtype != torch.bfloat16 or dw_into.stride(1) != 1):
            dh, dw, db = cuda_ops.linear_ce_bwd(dloss, h, w, bias, labels, lse)
            dw_into.add_(dw.to(dw_into.dtype))
            return dh, None, db
        return cuda_ops.linear_ce_bwd(dloss, h, w, bias, labels, lse, dw_into)
    logits = F.linear(h, w, bias).float()
    p = torch.exp(logits - lse[:, None])
    p[torch.arange(p.shape[0], device=p.device), labels] -= 1.0
    dlogits = (p * dloss.float()[:, None]).to(h.dtype)
    dh = dlogits @ w
    dw = dlogits.t() @ h
    db = dlogits.float().sum(0).to(bias.dtype) if bias is not None else None
    if dw_into is not None:
        dw_into.add_(dw.to(dw_into.dtype))
        dw = None
    return dh, dw, db
