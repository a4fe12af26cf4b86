"""Plain-PyTorch statements of every hot op.

These functions are the numerical oracle for the sm_100a kernels in ``csrc/`` and the
execution path on CPU (tests, gloo ranks).  They are written from the math contracts of
the reference model code (OpenTau ``src/opentau/utils/transformers_patch.py:68-167`` for the
norms and gated residual, ``policies/pi05/paligemma_with_expert.py:52-107,882-953`` for RoPE
and eager attention, ``policies/utils.py:283-354`` for the masked flow-matching MSE), not from
its code: everything is a free function over tensors, differentiable by autograd.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import Tensor

# Value the reference uses for masked logits (``paligemma_with_expert.py:930-940``): a large
# finite negative so that a fully masked row gives a uniform softmax instead of NaN.
BIG_NEG = -2.3819763e38
INT_MIN = -(2**31)


# ----------------------------------------------------------------------------- GEMM
def linear(x: Tensor, w: Tensor, bias: Tensor | None = None, residual: Tensor | None = None) -> Tensor:
    """``x @ w.T (+ bias) (+ residual)``; ``w`` is ``(out, in)`` like ``nn.Linear``."""
    y = F.linear(x, w, bias)
    if residual is not None:
        y = y + residual
    return y


# ----------------------------------------------------------------------------- norms
def rms_norm(x: Tensor, weight: Tensor | None, eps: float = 1e-6, unit_offset: bool = True) -> Tensor:
    """RMSNorm with the variance in fp32.

    ``unit_offset=True`` is Gemma's ``x * rsqrt(var+eps) * (1 + w)``; ``False`` is the
    Qwen/LLaMA ``w * x * rsqrt(var+eps)``.  ``weight=None`` applies no scale.
    """
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    y = xf * torch.rsqrt(var + eps)
    if weight is not None:
        y = y * ((1.0 + weight.float()) if unit_offset else weight.float())
    return y.to(x.dtype)


def ada_rms_norm(x: Tensor, mod: Tensor, eps: float = 1e-6) -> tuple[Tensor, Tensor]:
    """Adaptive RMSNorm: ``mod`` holds ``(scale, shift, gate)`` chunks along the last dim.

    Returns ``(normed * (1 + scale) + shift, gate)``.  ``mod`` is ``(B, 3H)`` (one condition
    per sample) or ``(B, S, 3H)`` (one per token).
    """
    if mod.dim() == x.dim() - 1:
        mod = mod.unsqueeze(-2)
    scale, shift, gate = mod.float().chunk(3, dim=-1)
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    y = xf * torch.rsqrt(var + eps)
    y = y * (1.0 + scale) + shift
    return y.to(x.dtype), gate.to(x.dtype)


def layer_norm(x: Tensor, weight: Tensor, bias: Tensor, eps: float = 1e-6) -> Tensor:
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), bias.float(), eps).to(x.dtype)


def gated_residual(x: Tensor, y: Tensor, gate: Tensor | None) -> Tensor:
    """``x + y * gate`` (``gate=None`` means a plain residual)."""
    if gate is None:
        return x + y
    return x + y * gate


# ----------------------------------------------------------------------------- rotary
def rope_angles(positions: Tensor, head_dim: int, theta: float) -> tuple[Tensor, Tensor]:
    """cos/sin tables ``(B, S, D/2)`` in fp32 for 1-D positions ``(B, S)``."""
    half = head_dim // 2
    frac = 2.0 * torch.arange(half, dtype=torch.float32, device=positions.device) / head_dim
    timescale = theta**frac
    ang = positions.float()[..., None] / timescale
    return torch.cos(ang), torch.sin(ang)


def mrope_angles(positions: Tensor, head_dim: int, theta: float, interleaved: bool = True,
                 sections: tuple[int, ...] | None = None) -> tuple[Tensor, Tensor]:
    """cos/sin for 3-axis positions ``(3, B, S)``.

    ``interleaved``: frequency band ``i`` is driven by axis ``i % 3`` (the pi05_mem / Qwen3-VL
    interleaved layout).  Otherwise ``sections`` gives contiguous band counts per axis.
    """
    half = head_dim // 2
    frac = 2.0 * torch.arange(half, dtype=torch.float32, device=positions.device) / head_dim
    timescale = theta**frac
    # built from device-side arithmetic only (no host tensor, no data-dependent size): safe inside a CUDA-graph capture
    ar = torch.arange(half, device=positions.device)
    if interleaved:
        axis = ar % 3
        if sections is not None:
            # Qwen3-VL: interleave only inside the first 3*min-section bands, rest use axis 0.
            lim = [3 * s for s in sections]
            axis = torch.zeros(half, dtype=torch.long, device=positions.device)
            for a in (1, 2):
                axis = torch.where((ar % 3 == a) & (ar < lim[a]), a, axis)
    else:
        assert sections is not None and sum(sections) == half
        axis = (ar >= sections[0]).long() + (ar >= sections[0] + sections[1]).long()
    pos = positions.float().permute(1, 2, 0)  # (B,S,3)
    sel = pos[..., axis]  # (B,S,half)
    ang = sel / timescale
    return torch.cos(ang), torch.sin(ang)


def apply_rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """Split-half rotation of ``x (B,S,H,D)`` by tables ``(B,S,D/2)``, computed in fp32."""
    d2 = x.shape[-1] // 2
    xf = x.float()
    x1, x2 = xf[..., :d2], xf[..., d2:]
    c, s = cos[:, :, None, :], sin[:, :, None, :]
    out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
    return out.to(x.dtype)


# ----------------------------------------------------------------------------- MLP
def glu_act(gate_up: Tensor, act: str = "gelu_tanh") -> Tensor:
    """``act(gate) * up`` for ``gate_up = [gate | up]`` concatenated on the last dim."""
    g, u = gate_up.chunk(2, dim=-1)
    if act == "gelu_tanh":
        a = F.gelu(g.float(), approximate="tanh")
    elif act == "silu":
        a = F.silu(g.float())
    else:
        raise ValueError(act)
    return (a * u.float()).to(gate_up.dtype)


def act_fn(x: Tensor, act: str) -> Tensor:
    if act == "gelu_tanh":
        return F.gelu(x.float(), approximate="tanh").to(x.dtype)
    if act == "silu":
        return F.silu(x.float()).to(x.dtype)
    if act == "gelu":
        return F.gelu(x.float()).to(x.dtype)
    raise ValueError(act)


# ----------------------------------------------------------------------------- attention
def make_block_ids(pad_masks: Tensor, att_masks: Tensor) -> tuple[Tensor, Tensor]:
    """Block-id codec of the 2-D mask rule ``cumsum(att)[j] <= cumsum(att)[i] & pad_i & pad_j``.

    Returns ``(blk int32 (B,S), valid bool (B,S))``.  Reference:
    ``policies/flash_attn_cuda/__init__.py:55-109`` and ``pi05/modeling_pi05.py:120-190``.
    """
    blk = torch.cumsum(att_masks.to(torch.int32), dim=1).to(torch.int32)
    return blk, pad_masks.to(torch.bool)


def dense_mask_from_blocks(q_blk: Tensor, k_blk: Tensor, q_valid: Tensor, k_valid: Tensor) -> Tensor:
    """bool ``(B, Sq, Sk)``: query i sees key j iff both valid and ``k_blk[j] <= q_blk[i]``."""
    return (k_blk[:, None, :] <= q_blk[:, :, None]) & q_valid[:, :, None] & k_valid[:, None, :]


def block_attention(q: Tensor, k: Tensor, v: Tensor, q_blk: Tensor, k_blk: Tensor,
                    q_valid: Tensor, k_valid: Tensor, scale: float) -> Tensor:
    """Block-causal GQA attention, token-major.

    ``q (B,Sq,H,D)``, ``k,v (B,Sk,Hkv,D)`` -> ``(B,Sq,H*D)``.  Logits and softmax in fp32,
    masked logits set to ``BIG_NEG``; rows with no visible key return zeros.
    """
    B, Sq, H, D = q.shape
    Hkv = k.shape[2]
    g = H // Hkv
    mask = dense_mask_from_blocks(q_blk, k_blk, q_valid, k_valid)  # (B,Sq,Sk)
    qf = q.float().view(B, Sq, Hkv, g, D)
    kf = k.float()
    s = torch.einsum("bqhgd,bkhd->bhgqk", qf, kf) * scale
    s = torch.where(mask[:, None, None], s, torch.full_like(s, BIG_NEG))
    p = torch.softmax(s, dim=-1)
    any_vis = mask.any(-1)[:, None, None, :, None]
    p = torch.where(any_vis, p, torch.zeros_like(p))
    o = torch.einsum("bhgqk,bkhd->bqhgd", p.to(v.dtype).float(), v.float())
    return o.reshape(B, Sq, H * D).to(q.dtype)


def mha(q: Tensor, k: Tensor, v: Tensor, scale: float, add_mask: Tensor | None = None) -> Tensor:
    """Unmasked (or additive-mask) multi-head attention ``(B,S,H,D)`` -> ``(B,S,H*D)``."""
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    if add_mask is not None:
        s = s + add_mask
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("bhqk,bkhd->bqhd", p, v.float())
    return o.reshape(q.shape[0], q.shape[1], -1).to(q.dtype)


# ----------------------------------------------------------------------------- losses
def flow_matching_masked_mse(u_t: Tensor, v_t: Tensor, prefix_mask: Tensor | None = None,
                             actions_is_pad: Tensor | None = None,
                             real_action_dim: Tensor | None = None,
                             return_per_sample: bool = False):
    """Masked MSE over ``(B, T, A)``: frozen-prefix steps, padded steps and padded action
    dims are excluded; denominator ``mask.sum() + 1e-8`` (``policies/utils.py:283-354``)."""
    B, T, A = u_t.shape
    mask = torch.ones(B, T, A, dtype=torch.bool, device=u_t.device)
    if prefix_mask is not None:
        mask &= ~prefix_mask.to(u_t.device)[:, :, None]
    if actions_is_pad is not None:
        mask &= ~actions_is_pad.to(torch.bool)[:, :, None]
    if real_action_dim is not None:
        dim = torch.arange(A, device=u_t.device)[None, None, :]
        mask &= dim < real_action_dim.view(B, 1, 1)
    se = (u_t.float() - v_t.float()).pow(2) * mask
    loss = se.sum() / (mask.sum() + 1e-8)
    if return_per_sample:
        return loss, (se.sum(dim=(1, 2)), mask.sum(dim=(1, 2)).float())
    return loss


def cross_entropy_tokens(logits: Tensor, labels: Tensor) -> Tensor:
    """Per-token CE with fp32 logits; ``logits (N,V)``, ``labels (N,)`` -> ``(N,)``."""
    return F.cross_entropy(logits.float(), labels, reduction="none")


def linear_cross_entropy(h: Tensor, w: Tensor, bias: Tensor | None, labels: Tensor) -> Tensor:
    """``CE(h @ w.T + b, labels)`` per row with fp32 logits."""
    logits = F.linear(h, w, bias).float()
    return F.cross_entropy(logits, labels, reduction="none")


# ----------------------------------------------------------------------------- flow matching
def sinusoidal_time_embedding(time: Tensor, dim: int, min_period: float = 4e-3,
                              max_period: float = 4.0) -> Tensor:
    """``[sin | cos]`` embedding of scalar times ``(B,T)`` -> ``(B,T,dim)`` (fp32 out).

    Periods are log-spaced between ``min_period`` and ``max_period``
    (``pi05/modeling_pi05.py:81-117``); computed in fp64 on CPU, fp32 on device.
    """
    dt = torch.float64 if time.device.type == "cpu" else torch.float32
    frac = torch.linspace(0.0, 1.0, dim // 2, dtype=dt, device=time.device)
    period = min_period * (max_period / min_period) ** frac
    ang = (2 * math.pi / period)[None, None, :] * time.to(dt)[:, :, None]
    return torch.cat([torch.sin(ang), torch.cos(ang)], dim=2).float()


def flow_interpolate(actions: Tensor, noise: Tensor, time: Tensor) -> tuple[Tensor, Tensor]:
    """``x_t = t*eps + (1-t)*a``, ``u_t = eps - a`` with ``time (B,T)``."""
    t = time[:, :, None]
    return t * noise + (1 - t) * actions, noise - actions


# ----------------------------------------------------------------------------- images
def resize_with_pad(img: Tensor, width: int, height: int, pad_value: float = -1.0) -> Tensor:
    """Aspect-preserving bilinear resize (``align_corners=False``) then pad on the left/top.

    ``img (B,C,H,W)``.  Mirrors ``pi05/modeling_pi05.py:193-232`` behaviour.
    """
    if img.ndim != 4:
        raise ValueError(f"(b,c,h,w) expected, got {tuple(img.shape)}")
    ch, cw = img.shape[2:]
    ratio = max(cw / width, ch / height)
    rh, rw = int(ch / ratio), int(cw / ratio)
    out = F.interpolate(img, size=(rh, rw), mode="bilinear", align_corners=False)
    ph, pw = max(0, height - rh), max(0, width - rw)
    return F.pad(out, (pw, 0, ph, 0), value=pad_value)


# ----------------------------------------------------------------------------- optimizer
def adamw_flat(p32: Tensor, g: Tensor, m: Tensor, v: Tensor, p16: Tensor | None, *, lr: float,
               beta1: float, beta2: float, eps: float, weight_decay: float, step: int,
               grad_scale: float = 1.0) -> None:
    """In-place decoupled AdamW on flat fp32 masters; optionally refreshes the bf16 copy.

    ``g`` may be bf16 or fp32 and is multiplied by ``grad_scale`` (mean over ranks x clip
    coefficient) before use.  Matches ``torch.optim.AdamW`` update order.
    """
    gf = g.float() * grad_scale
    p32.mul_(1.0 - lr * weight_decay)
    m.mul_(beta1).add_(gf, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1.0 - beta2)
    bc1 = 1.0 - beta1**step
    bc2 = 1.0 - beta2**step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p32.addcdiv_(m, denom, value=-lr / bc1)
    if p16 is not None:
        p16.copy_(p32)
