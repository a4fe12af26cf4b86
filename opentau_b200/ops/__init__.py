"""Public op surface of the framework.

``ops.<name>`` is what model code calls.  Each differentiable op is a hand-written
autograd function (``fused.py``) over single-launch primitives (``prims.py``); a primitive
runs the sm_100a kernel for CUDA bf16 tensors and a plain-PyTorch body on CPU.  Setting
``OPENTAU_B200_ORACLE=1`` routes everything to ``reference.py`` (plain autograd over library
calls) — the comparison arm, never the product path.  On a CUDA tensor a missing native
library raises; there is no silent fallback.
"""

from __future__ import annotations

import os

from torch import Tensor


def oracle_mode() -> bool:
    return os.environ.get("OPENTAU_B200_ORACLE", "0") == "1"


from . import reference as ref  # noqa: E402
from .reference import (BIG_NEG, INT_MIN, apply_rope, dense_mask_from_blocks, make_block_ids,  # noqa: E402
                        mrope_angles, rope_angles)
from . import prims, fused  # noqa: E402


def linear(x: Tensor, w: Tensor, bias: Tensor | None = None, residual: Tensor | None = None) -> Tensor:
    if oracle_mode():
        return ref.linear(x, w, bias, residual)
    return fused.linear(x, w, bias, residual)


def rms_norm(x: Tensor, weight: Tensor | None, eps: float = 1e-6, unit_offset: bool = True) -> Tensor:
    if oracle_mode():
        return ref.rms_norm(x, weight, eps, unit_offset)
    return fused.rms_norm(x, weight, eps, unit_offset)


def ada_rms_norm(x: Tensor, mod: Tensor, eps: float = 1e-6):
    if oracle_mode():
        return ref.ada_rms_norm(x, mod, eps)
    return fused.ada_rms_norm(x, mod, eps)


def rms_norm_fork(x: Tensor, weight: Tensor | None, eps: float = 1e-6, unit_offset: bool = True):
    """``(norm(x), x_res)``: use ``x_res`` (the same values as ``x``) for the residual connection around the normalised
    branch, so that the backward adds the residual gradient inside the norm's backward kernel."""
    import torch
    if oracle_mode() or not (torch.is_grad_enabled() and x.requires_grad):
        return rms_norm(x, weight, eps, unit_offset), x
    return fused.rms_norm_fork(x, weight, eps, unit_offset)


def ada_rms_norm_fork(x: Tensor, mod: Tensor, eps: float = 1e-6):
    """Adaptive form of :func:`rms_norm_fork`: ``(y, gate, x_res)``."""
    import torch
    if oracle_mode() or not (torch.is_grad_enabled() and x.requires_grad):
        y, gate = ada_rms_norm(x, mod, eps)
        return y, gate, x
    return fused.ada_rms_norm_fork(x, mod, eps)


def layer_norm(x: Tensor, weight: Tensor, bias: Tensor, eps: float = 1e-6) -> Tensor:
    if oracle_mode():
        return ref.layer_norm(x, weight, bias, eps)
    return fused.layer_norm(x, weight, bias, eps)


def patch_embed(pixels: Tensor, weight: Tensor, bias: Tensor, pos: Tensor, patch: int, out_dtype) -> Tensor:
    """Non-overlapping patch convolution + bias + position table, computed in fp32 and cast to ``out_dtype``:
    ``pixels (B,C,H,W)`` with ``H, W`` multiples of ``patch``, ``weight (N,C,p,p)``, ``pos (gh*gw, N)``."""
    import torch
    import torch.nn.functional as F
    if pixels.is_cuda and not oracle_mode() and not (torch.is_grad_enabled() and pixels.requires_grad):
        return fused.patch_embed(pixels, weight, bias, pos, patch, out_dtype)
    B, C, H, W = pixels.shape
    gh, gw = H // patch, W // patch
    x = pixels.float().view(B, C, gh, patch, gw, patch).permute(0, 2, 4, 1, 3, 5).reshape(B, gh * gw, C * patch * patch)
    y = F.linear(x, weight.float().view(weight.shape[0], -1), bias.float()) + pos.float()
    return y.to(out_dtype)


def sinusoidal_time_embedding(time: Tensor, dim: int, min_period: float = 4e-3, max_period: float = 4.0,
                              out_dtype=None) -> Tensor:
    """``[sin | cos]`` embedding of scalar times ``(B,T) -> (B,T,dim)`` (fp32 unless ``out_dtype`` says otherwise): one
    kernel on CUDA, the fp64 / fp32 statement of ``reference.py`` elsewhere."""
    import torch
    if time.is_cuda and not oracle_mode() and not time.requires_grad and time.dim() == 2:
        from . import cuda_ops
        return cuda_ops.time_embed(time, dim, min_period, max_period, out_dtype or torch.float32)
    e = ref.sinusoidal_time_embedding(time, dim, min_period, max_period)
    return e.to(out_dtype) if out_dtype is not None else e


def flow_interpolate(actions: Tensor, noise: Tensor, time: Tensor):
    """``x_t = t*eps + (1-t)*a``, ``u_t = eps - a`` with ``time (B,T)``; one kernel on CUDA when nothing needs a
    gradient (actions and noise are data)."""
    import torch
    if actions.is_cuda and not oracle_mode() and actions.shape == noise.shape and time.shape == actions.shape[:2] \
            and not (torch.is_grad_enabled() and (actions.requires_grad or noise.requires_grad or time.requires_grad)):
        from . import cuda_ops
        return cuda_ops.flow_interpolate(actions, noise, time)
    return ref.flow_interpolate(actions, noise, time)


def euler_step(x_t: Tensor, v_t: Tensor, dt: float, frozen: Tensor | None = None,
               action_prefix: Tensor | None = None) -> Tensor:
    """One Euler step of the flow ODE, ``x_t + dt * v_t``, with rows of a committed action prefix (``frozen (B,T)``)
    held at ``action_prefix``.  On CUDA the fp32 sample is updated in place by one kernel."""
    import torch
    if x_t.is_cuda and not oracle_mode() and x_t.dtype == torch.float32 and x_t.is_contiguous() \
            and not torch.is_grad_enabled():
        from . import cuda_ops
        return cuda_ops.euler_step_(x_t, v_t, dt, frozen if action_prefix is not None else None, action_prefix)
    x = x_t + dt * v_t.to(x_t.dtype)
    if action_prefix is not None and frozen is not None:
        x = torch.where(frozen[:, :, None], action_prefix.to(x.dtype), x)
    return x


def _native_nograd(*ts: Tensor) -> bool:
    """Inference fusions: CUDA bf16 tensors, nothing to differentiate, not the oracle arm."""
    import torch
    return (not oracle_mode() and ts[0].is_cuda and ts[0].dtype == torch.bfloat16
            and not (torch.is_grad_enabled() and any(t.requires_grad for t in ts if t is not None)))


def gated_residual(x: Tensor, y: Tensor, gate: Tensor | None) -> Tensor:
    if gate is not None and x.dim() == 3 and _native_nograd(x, y, gate) and x.shape[-1] % 8 == 0 \
            and gate.dtype == x.dtype and y.dtype == x.dtype:
        from . import cuda_ops
        return cuda_ops.gated_residual(x, y, gate)
    return ref.gated_residual(x, y, gate)


def _gate_rows(gate: Tensor, x: Tensor):
    """``gate (B,1,H) | (B,T,H)`` as 2-D rows for the GEMM epilogue, or None when it cannot be passed as is."""
    g = gate.reshape(-1, gate.shape[-1])
    if g.dtype != x.dtype or g.stride(1) != 1 or g.stride(0) % 8 or g.data_ptr() % 16:
        return None
    rows = x.shape[0] * x.shape[1]
    return g if rows % g.shape[0] == 0 else None


def linear_gated_residual(x: Tensor, w: Tensor, bias: Tensor | None, residual: Tensor, gate: Tensor | None) -> Tensor:
    """``residual + gate * linear(x)``.  At inference with few rows the gate and the residual are applied in the
    epilogue of the projection (one launch); otherwise projection and gated residual run separately."""
    if gate is not None and x.dim() == 3 and _native_nograd(x, w, residual, gate):
        from . import cuda_ops
        rows, g2 = x.shape[0] * x.shape[1], _gate_rows(gate, x)
        if g2 is not None and cuda_ops.use_skinny("nt", rows, w.shape[0], False, 0) and w.shape[0] % 8 == 0 \
                and x.shape[-1] % 8 == 0:
            out = cuda_ops.gemm(x.reshape(rows, -1), w, "nt", bias=bias, residual=residual.reshape(rows, -1).contiguous(),
                                gate=g2)
            return out.view(*x.shape[:-1], w.shape[0])
    return gated_residual(residual, linear(x, w, bias), gate)


def gated_mlp_gated_residual(x: Tensor, w_gate_up: Tensor, w_down: Tensor, act: str, residual: Tensor,
                             gate: Tensor | None) -> Tensor:
    """``residual + gate * down(act(gate_proj x) * up_proj x)`` with the same epilogue fusion at inference."""
    if gate is not None and x.dim() == 3 and _native_nograd(x, w_gate_up, residual, gate):
        from . import cuda_ops
        rows, g2 = x.shape[0] * x.shape[1], _gate_rows(gate, x)
        if g2 is not None and cuda_ops.use_skinny("nt", rows, w_down.shape[0], False, 0) \
                and cuda_ops.use_skinny("nt", rows, w_gate_up.shape[0], False, 0):
            h = cuda_ops.gemm(x.reshape(rows, -1), w_gate_up, "nt", glu=act, store_out=False)
            out = cuda_ops.gemm(h, w_down, "nt", residual=residual.reshape(rows, -1).contiguous(), gate=g2)
            return out.view(*x.shape[:-1], w_down.shape[0])
    return gated_residual(residual, gated_mlp(x, w_gate_up, w_down, act), gate)


def qkv_post(qkv: Tensor, heads: int, kv_heads: int, head_dim: int, q_norm, k_norm, cos: Tensor, sin: Tensor,
             k_dst: Tensor | None = None, v_dst: Tensor | None = None):
    """Inference-only fusion after the q/k/v projection of one tower: split, optional per-head RMSNorm of q and k
    (``q_norm / k_norm``: modules with ``weight, eps, unit_offset``, or None), rotation of q and k, and the store of k
    and v, optionally straight into ``k_dst / v_dst`` (strided ``(B,T,Hkv,D)`` views, e.g. the tail of a KV cache).
    Returns ``(q (B,T,H,D), k, v)``."""
    from . import cuda_ops
    return cuda_ops.qkv_post(qkv, heads, kv_heads, head_dim, q_norm, k_norm, cos, sin, k_dst, v_dst)


def can_fuse_qkv_post(x: Tensor, head_dim: int) -> bool:
    return _native_nograd(x) and head_dim % 8 == 0 and head_dim <= 256


def rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    if oracle_mode():
        return ref.apply_rope(x, cos, sin)
    return fused.rope(x, cos, sin)


def gated_mlp(x: Tensor, w_gate_up: Tensor, w_down: Tensor, act: str, residual: Tensor | None = None) -> Tensor:
    """``down(act(gate)·up)`` with the block-interleaved fused gate/up weight (``prims.GLU_BLOCK``)."""
    if oracle_mode():
        gu = ref.linear(x, w_gate_up)
        h = _ref_glu(gu, act)
        return ref.linear(h, w_down, None, residual)
    return fused.gated_mlp(x, w_gate_up, w_down, act, residual)


def _ref_glu(gu: Tensor, act: str) -> Tensor:
    g, u = prims._split_glu(gu)
    return (ref.act_fn(g.float(), act) * u.float()).flatten(-2).to(gu.dtype)


def act_fn(x: Tensor, act: str) -> Tensor:
    return ref.act_fn(x, act)


def linear_act(x: Tensor, w: Tensor, bias: Tensor | None, act: str) -> Tensor:
    """``act(x @ w.T + bias)``; when no gradient is needed the activation runs in the GEMM epilogue."""
    import torch
    needs_grad = torch.is_grad_enabled() and (x.requires_grad or w.requires_grad)
    if (not oracle_mode() and not needs_grad and x.is_cuda and x.dtype == torch.bfloat16 and act == "gelu_tanh"):
        from . import cuda_ops
        y = cuda_ops.gemm(x.reshape(-1, x.shape[-1]), w, "nt", bias=bias, act="gelu_tanh")
        return y.view(*x.shape[:-1], w.shape[0])
    return ref.act_fn(linear(x, w, bias), act)


def block_attention(q: Tensor, k: Tensor, v: Tensor, q_blk: Tensor, k_blk: Tensor,
                    q_valid: Tensor, k_valid: Tensor, scale: float) -> Tensor:
    if oracle_mode():
        return ref.block_attention(q, k, v, q_blk, k_blk, q_valid, k_valid, scale)
    return fused.block_attention(q, k, v, q_blk, k_blk, q_valid, k_valid, scale)


def mha(q: Tensor, k: Tensor, v: Tensor, scale: float, add_mask: Tensor | None = None) -> Tensor:
    """Full (unmasked) multi-head attention; with ``add_mask`` it stays on the reference body."""
    if oracle_mode() or add_mask is not None:
        return ref.mha(q, k, v, scale, add_mask)
    import torch
    B, S, _, _ = q.shape
    Sk = k.shape[1]
    zq = torch.zeros(B, S, dtype=torch.int32, device=q.device)
    zk = torch.zeros(B, Sk, dtype=torch.int32, device=q.device)
    oq = torch.ones(B, S, dtype=torch.bool, device=q.device)
    ok = torch.ones(B, Sk, dtype=torch.bool, device=q.device)
    return fused.block_attention(q, k, v, zq, zk, oq, ok, scale)


def flow_matching_masked_mse(u_t, v_t, prefix_mask=None, actions_is_pad=None, real_action_dim=None,
                             return_per_sample=False):
    if u_t.is_cuda and not oracle_mode():
        loss, sums, counts = fused.MaskedMSEFn.apply(u_t, v_t, prefix_mask, actions_is_pad, real_action_dim)
        return (loss, (sums, counts)) if return_per_sample else loss
    return ref.flow_matching_masked_mse(u_t, v_t, prefix_mask, actions_is_pad, real_action_dim,
                                        return_per_sample)


def dropout_gated_residual(x: Tensor, y: Tensor, gate: Tensor | None, p: float, training: bool) -> Tensor:
    """``x + gate * dropout(y, p)`` (``gate=None``: plain residual).  The reference applies ``nn.Dropout`` after the
    attention output projection and after the MLP, then the (gated) residual
    (``pi05/paligemma_with_expert.py:783-792``); on the GPU the three are one kernel in each direction."""
    import torch
    if not training or p <= 0.0:
        return gated_residual(x, y, gate)
    if (x.is_cuda and not oracle_mode() and x.dtype == torch.bfloat16 and y.dtype == x.dtype and x.dim() == 3
            and x.shape[-1] % 8 == 0 and (gate is None or (gate.dtype == x.dtype and gate.dim() == 3 and (
                x.shape[0] * x.shape[1]) % (gate.shape[0] * gate.shape[1]) == 0 and gate.shape[0] == x.shape[0]))):
        return fused.dropout_residual(x, y, gate, p)
    return gated_residual(x, torch.nn.functional.dropout(y, p, True), gate)


def embedding(table: Tensor, ids: Tensor, scale: float = 1.0, padding_idx: int | None = None) -> Tensor:
    """``table[ids] * scale``: gather kernel forward, deterministic scatter-add backward (no dense one-hot product,
    no atomics; row ``padding_idx`` takes no gradient); plain indexing on the CPU / in oracle mode."""
    import torch
    if table.is_cuda and not oracle_mode() and table.dtype == torch.bfloat16 and table.shape[1] % 8 == 0:
        if torch.is_grad_enabled() and table.requires_grad:
            return fused.embedding(table, ids, scale, padding_idx)
        from . import cuda_ops
        return cuda_ops.embed_fwd(table, ids, scale)
    out = torch.nn.functional.embedding(ids, table, padding_idx=padding_idx)
    return out * scale if scale != 1.0 else out


def seq_concat(a: Tensor, c: Tensor) -> Tensor:
    """``cat([a, c], dim=1)``: cached keys / values followed by the new ones.  One copy kernel for dense bf16 rows on
    the GPU, ``torch.cat`` otherwise."""
    import torch
    if a.is_cuda and not oracle_mode():
        from . import cuda_ops
        if cuda_ops.seq_concat_supported(a, c):
            if torch.is_grad_enabled() and (a.requires_grad or c.requires_grad):
                return fused.SeqConcatFn.apply(a, c)
            return cuda_ops.seq_concat(a, c)
    return torch.cat([a, c], dim=1)


def linear_cross_entropy(h: Tensor, w: Tensor, bias: Tensor | None, labels: Tensor) -> Tensor:
    if oracle_mode():
        return ref.linear_cross_entropy(h, w, bias, labels)
    return fused.linear_cross_entropy(h, w, bias, labels)


def resize_with_pad(img: Tensor, width: int, height: int, pad_value: float = -1.0) -> Tensor:
    if img.is_cuda and not oracle_mode():
        from . import cuda_ops
        return cuda_ops.resize_with_pad(img, width, height, pad_value)
    return ref.resize_with_pad(img, width, height, pad_value)


__all__ = [
    "BIG_NEG", "INT_MIN", "linear", "rms_norm", "ada_rms_norm", "layer_norm", "gated_residual", "linear_gated_residual", "gated_mlp_gated_residual", "qkv_post", "can_fuse_qkv_post", "rope",
    "gated_mlp", "act_fn", "linear_act", "block_attention", "mha", "flow_matching_masked_mse", "linear_cross_entropy",
    "resize_with_pad", "dropout_gated_residual", "embedding", "make_block_ids", "dense_mask_from_blocks", "rope_angles", "mrope_angles",
    "apply_rope", "rms_norm_fork", "ada_rms_norm_fork", "seq_concat", "sinusoidal_time_embedding", "flow_interpolate", "euler_step", "patch_embed", "oracle_mode", "prims", "fused", "ref",
]
