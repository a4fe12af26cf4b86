"""Autograd functions whose forward and backward are explicit sequences of primitives.

Writing the backward by hand (instead of letting autograd chain small ops) is what lets each
step be one fused kernel on the B200 and lets the MLP keep only ``x`` and the gate/up GEMM
output alive between forward and backward.

Weight gradients: when a parameter carries a ``main_grad`` tensor (a view into the flat
gradient buffer of ``parallel.flat.FlatParamStore``) the weight-gradient GEMM accumulates
straight into it and autograd receives ``None``; otherwise the gradient is returned normally.
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import prims


# Called with a parameter every time a backward pass has QUEUED the last kernel that writes that parameter's
# ``main_grad`` for one use of the parameter.  The training engine hangs its bucketed gradient reduction on it.
_grad_ready_hook = None


def set_grad_ready_hook(fn) -> None:
    global _grad_ready_hook
    _grad_ready_hook = fn


def _notify(pref) -> None:
    if _grad_ready_hook is not None:
        _grad_ready_hook(pref)


def _flat2d(x: Tensor) -> Tensor:
    return x.reshape(-1, x.shape[-1])


def _sink_wgrad(wref, a: Tensor, b: Tensor):
    """d(weight) = a.T @ b, into ``main_grad`` when present (returns None) else returned."""
    mg = getattr(wref, "main_grad", None)
    if mg is not None:
        prims.mm_tn(a, b, out=mg, accumulate=True)
        _notify(wref)
        return None
    return prims.mm_tn(a, b)


def _sink_vec(pref, g: Tensor):
    mg = getattr(pref, "main_grad", None)
    if mg is not None:
        mg.add_(g.to(mg.dtype))
        _notify(pref)
        return None
    return g


class LinearFn(torch.autograd.Function):
    """``y = x @ w.T (+ bias) (+ residual)``."""

    @staticmethod
    def forward(ctx, x, w, bias, residual):
        x2 = _flat2d(x)
        r2 = _flat2d(residual) if residual is not None else None
        y = prims.mm_nt(x2, w, bias=bias, residual=r2)
        ctx.save_for_backward(x2, w)
        ctx.wref, ctx.bref = w, bias
        ctx.x_shape = x.shape
        ctx.has_res = residual is not None
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _flat2d(dy)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = prims.mm_nn(dy2, w).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            dw = _sink_wgrad(ctx.wref, dy2, x2)
        if ctx.bref is not None and ctx.needs_input_grad[2]:
            db = _sink_vec(ctx.bref, prims.col_sum(dy2))
        dres = dy if ctx.has_res else None
        return dx, dw, db, dres


def linear(x, w, bias=None, residual=None):
    return LinearFn.apply(x, w, bias, residual)


class GatedMLPFn(torch.autograd.Function):
    """``down(act(gate(x)) * up(x)) (+ residual)`` with a fused, block-interleaved gate/up weight.

    The activation product comes out of the gate/up GEMM's epilogue.  For the backward ``x``, the gate/up
    output and the product are kept (180 GB of HBM make the recompute pointless); the gradient of the
    gate/up output overwrites that buffer in place.
    """

    @staticmethod
    def forward(ctx, x, w_gu, w_down, residual, act):
        x2 = _flat2d(x)
        need_bwd = any(ctx.needs_input_grad[:3])
        gu, h = prims.mm_nt_glu(x2, w_gu, act, keep_gu=need_bwd)
        r2 = _flat2d(residual) if residual is not None else None
        y = prims.mm_nt(h, w_down, residual=r2)
        if need_bwd:
            ctx.save_for_backward(x2, gu, h, w_gu, w_down)
        ctx.wgu, ctx.wdown = w_gu, w_down
        ctx.act, ctx.x_shape, ctx.has_res = act, x.shape, residual is not None
        return y.view(*x.shape[:-1], w_down.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, gu, h, w_gu, w_down = ctx.saved_tensors
        dy2 = _flat2d(dy)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dwd = _sink_wgrad(ctx.wdown, dy2, h) if ctx.needs_input_grad[2] else None
        dh = prims.mm_nn(dy2, w_down, out=h)  # h is dead after the weight gradient
        dgu = prims.glu_bwd(gu, dh, ctx.act, inplace=True)
        del dh, h
        dwgu = _sink_wgrad(ctx.wgu, dgu, x2) if ctx.needs_input_grad[1] else None
        dx = prims.mm_nn(dgu, w_gu).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        return dx, dwgu, dwd, (dy if ctx.has_res else None), None


def gated_mlp(x, w_gu, w_down, act, residual=None):
    return GatedMLPFn.apply(x, w_gu, w_down, residual, act)


class RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, unit_offset):
        y, rstd = prims.rms_fwd(x, w, eps, unit_offset)
        ctx.save_for_backward(x, w if w is not None else x.new_empty(0), rstd)
        ctx.has_w, ctx.unit_offset, ctx.wref = w is not None, unit_offset, w
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dx, dw = prims.rms_bwd(dy.contiguous(), x, w if ctx.has_w else None, rstd, ctx.unit_offset)
        if dw is not None:
            dw = _sink_vec(ctx.wref, dw) if ctx.needs_input_grad[1] else None
        return dx, dw, None, None


def rms_norm(x, w, eps=1e-6, unit_offset=True):
    return RMSNormFn.apply(x, w, eps, unit_offset)


class RMSNormForkFn(torch.autograd.Function):
    """``x -> (norm(x), x)``: the second output is ``x`` itself, to be used by the residual connection around the
    normalised branch.  The two gradients that reach ``x`` (through the norm and through the residual) then arrive at
    ONE backward, which adds the residual gradient inside the norm's backward kernel instead of leaving the sum to a
    separate element-wise launch over the whole residual stream."""

    @staticmethod
    def forward(ctx, x, w, eps, unit_offset):
        y, rstd = prims.rms_fwd(x, w, eps, unit_offset)
        ctx.save_for_backward(x, w if w is not None else x.new_empty(0), rstd)
        ctx.has_w, ctx.unit_offset, ctx.wref = w is not None, unit_offset, w
        return y, x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dres):
        x, w, rstd = ctx.saved_tensors
        if dy is None:
            return dres, None, None, None
        dx, dw = prims.rms_bwd(dy.contiguous(), x, w if ctx.has_w else None, rstd, ctx.unit_offset, dres)
        if dw is not None:
            dw = _sink_vec(ctx.wref, dw) if ctx.needs_input_grad[1] else None
        return dx, dw, None, None


def rms_norm_fork(x, w, eps=1e-6, unit_offset=True):
    return RMSNormForkFn.apply(x, w, eps, unit_offset)


class AdaRMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mod, eps):
        y, rstd = prims.ada_rms_fwd(x, mod, eps)
        ctx.save_for_backward(x, mod, rstd)
        H = x.shape[-1]
        gate = mod[..., 2 * H:]
        if gate.dim() == 2:
            gate = gate[:, None, :]
        return y, gate

    @staticmethod
    def backward(ctx, dy, dgate):
        x, mod, rstd = ctx.saved_tensors
        dx, dscale, dshift = prims.ada_rms_bwd(dy.contiguous(), x, mod, rstd)
        if dgate is None:
            dgate = torch.zeros_like(dscale)
        elif mod.dim() == 2:
            dgate = dgate.reshape(mod.shape[0], -1, dscale.shape[-1]).sum(1) if dgate.dim() == 3 else dgate
        dmod = torch.cat([dscale, dshift, dgate.to(dscale.dtype)], dim=-1)
        return dx, dmod, None


def ada_rms_norm(x, mod, eps=1e-6):
    return AdaRMSNormFn.apply(x, mod, eps)


class AdaRMSNormForkFn(torch.autograd.Function):
    """Adaptive form of :class:`RMSNormForkFn`: ``x, mod -> (y, gate, x)``."""

    @staticmethod
    def forward(ctx, x, mod, eps):
        y, rstd = prims.ada_rms_fwd(x, mod, eps)
        ctx.save_for_backward(x, mod, rstd)
        H = x.shape[-1]
        gate = mod[..., 2 * H:]
        if gate.dim() == 2:
            gate = gate[:, None, :]
        return y, gate, x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dgate, dres):
        x, mod, rstd = ctx.saved_tensors
        if dy is None:
            dy = torch.zeros_like(x)
        dx, dscale, dshift = prims.ada_rms_bwd(dy.contiguous(), x, mod, rstd, dres)
        if dgate is None:
            dgate = torch.zeros_like(dscale)
        elif mod.dim() == 2:
            dgate = dgate.reshape(mod.shape[0], -1, dscale.shape[-1]).sum(1) if dgate.dim() == 3 else dgate
        dmod = torch.cat([dscale, dshift, dgate.to(dscale.dtype)], dim=-1)
        return dx, dmod, None


def ada_rms_norm_fork(x, mod, eps=1e-6):
    return AdaRMSNormForkFn.apply(x, mod, eps)


class LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        y, mean, rstd = prims.ln_fwd(x, w, b, eps)
        ctx.save_for_backward(x, w, mean, rstd)
        ctx.wref, ctx.bref = w, b
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, mean, rstd = ctx.saved_tensors
        dx, dw, db = prims.ln_bwd(dy.contiguous(), x, w, mean, rstd)
        return dx, _sink_vec(ctx.wref, dw), _sink_vec(ctx.bref, db), None


def layer_norm(x, w, b, eps=1e-6):
    return LayerNormFn.apply(x, w, b, eps)


class RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        ctx.save_for_backward(cos, sin)
        return prims.rope_fwd(x, cos, sin, inverse=False)

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        return prims.rope_fwd(dy, cos, sin, inverse=True), None, None


def rope(x, cos, sin):
    return RopeFn.apply(x, cos, sin)


class BlockAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, q_blk, k_blk, q_valid, k_valid, scale):
        o, lse = prims.attn_fwd(q, k, v, q_blk, k_blk, q_valid, k_valid, scale)
        ctx.save_for_backward(q, k, v, o, lse, q_blk, k_blk, q_valid, k_valid)
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, q_blk, k_blk, q_valid, k_valid = ctx.saved_tensors
        dq, dk, dv = prims.attn_bwd(do.contiguous(), q, k, v, o, lse, q_blk, k_blk, q_valid, k_valid, ctx.scale)
        return dq, dk, dv, None, None, None, None, None


def block_attention(q, k, v, q_blk, k_blk, q_valid, k_valid, scale):
    return BlockAttentionFn.apply(q, k, v, q_blk, k_blk, q_valid, k_valid, scale)


class LinearCEFn(torch.autograd.Function):
    """Per-row ``CE(h @ w.T + b, labels)`` without keeping the logits for the backward."""

    @staticmethod
    def forward(ctx, h, w, bias, labels):
        loss, lse = prims.linear_ce_fwd(h, w, bias, labels)
        ctx.save_for_backward(h, w, labels, lse)
        ctx.wref, ctx.bref = w, bias
        return loss

    @staticmethod
    def backward(ctx, dloss):
        h, w, labels, lse = ctx.saved_tensors
        mg = getattr(ctx.wref, "main_grad", None)
        dh, dw, db = prims.linear_ce_bwd(dloss.contiguous(), h, w, ctx.bref, labels, lse, dw_into=mg)
        if mg is not None:
            _notify(ctx.wref)
            dw = None
        if db is not None:
            db = _sink_vec(ctx.bref, db)
        return dh, dw, db, None


def linear_cross_entropy(h, w, bias, labels):
    return LinearCEFn.apply(h, w, bias, labels)



class PatchEmbedFn(torch.autograd.Function):
    """SigLIP patch embedding: forward is one native kernel (gather + fp32 product + bias + position table + cast);
    the backward needs only parameter gradients (pixels are data) and states them with library calls on the unfolded
    patches: three reductions per step, outside the forward hot path."""

    @staticmethod
    def forward(ctx, pixels, weight, bias, pos, patch, out_dtype):
        from . import cuda_ops
        ctx.save_for_backward(pixels)
        ctx.patch = patch
        return cuda_ops.patch_embed(pixels, weight.reshape(weight.shape[0], -1), bias, pos, patch, out_dtype)

    @staticmethod
    def backward(ctx, dy):
        (pixels,) = ctx.saved_tensors
        p = ctx.patch
        B, C, H, W = pixels.shape
        gh, gw = H // p, W // p
        g = dy.float()
        dw = db = dpos = None
        if ctx.needs_input_grad[1]:
            x = pixels.float().view(B, C, gh, p, gw, p).permute(0, 2, 4, 1, 3, 5).reshape(B * gh * gw, C * p * p)
            dw = (g.reshape(B * gh * gw, -1).t() @ x).view(-1, C, p, p)
        if ctx.needs_input_grad[2]:
            db = g.sum(dim=(0, 1))
        if ctx.needs_input_grad[3]:
            dpos = g.sum(dim=0)
        return None, dw, db, dpos, None, None


def patch_embed(pixels, weight, bias, pos, patch, out_dtype):
    return PatchEmbedFn.apply(pixels, weight, bias, pos, patch, out_dtype)


class DropoutResidualFn(torch.autograd.Function):
    """``x + gate * dropout(y, p)`` in one native pass each way; the keep mask is regenerated from the call's seed in
    the backward (nothing but the seed is kept for it; ``y`` only when a gate needs its gradient)."""

    @staticmethod
    def forward(ctx, x, y, gate, p: float):
        from . import cuda_ops
        seed = int(torch.randint(0, 2**62, (1,), device="cpu").item())      # from the host generator (seedable)
        out = cuda_ops.dropout_residual_fwd(x, y, gate, p, seed)
        ctx.p, ctx.seed = p, seed
        ctx.has_gate = gate is not None
        ctx.gate_shape = gate.shape if gate is not None else None
        ctx.save_for_backward(*( (y, gate) if gate is not None else () ))
        return out

    @staticmethod
    def backward(ctx, dout):
        from . import cuda_ops
        y, gate = ctx.saved_tensors if ctx.has_gate else (None, None)
        dy, dgate = cuda_ops.dropout_residual_bwd(dout, y, gate, ctx.p, ctx.seed)
        if dgate is not None:
            dgate = dgate.view(ctx.gate_shape).to(gate.dtype)
        return dout, dy, dgate, None


def dropout_residual(x, y, gate, p: float):
    return DropoutResidualFn.apply(x, y, gate, p)


class MaskedMSEFn(torch.autograd.Function):
    """Flow-matching masked MSE: per-sample sums and counts in one native pass; the backward writes the gradient of
    the prediction directly."""

    @staticmethod
    def forward(ctx, u, v, frozen, pad, real_dim):
        from . import cuda_ops
        u32, v32 = u.float().contiguous(), v.float().contiguous()
        fz = frozen.to(torch.uint8).contiguous() if frozen is not None else None
        pd = pad.to(torch.uint8).contiguous() if pad is not None else None
        rd = real_dim.to(torch.int64).contiguous() if real_dim is not None else None
        sums, counts = cuda_ops.masked_mse_fwd(u32, v32, fz, pd, rd)
        total = counts.sum() + 1e-8
        ctx.save_for_backward(u32, v32, total)
        ctx.masks = (fz, pd, rd)
        ctx.mark_non_differentiable(sums, counts)
        return sums.sum() / total, sums, counts

    @staticmethod
    def backward(ctx, dloss, _ds, _dc):
        from . import cuda_ops
        u32, v32, total = ctx.saved_tensors
        coef = (dloss.float() / total).reshape(1).contiguous()
        dv = cuda_ops.masked_mse_bwd(u32, v32, *ctx.masks, coef)
        return None, dv, None, None, None


class EmbeddingFn(torch.autograd.Function):
    """``table[ids] * scale`` with a gather kernel forward and a sort-by-id scatter-add backward that goes straight
    into the parameter's flat gradient (``main_grad``) when there is one."""

    @staticmethod
    def forward(ctx, table, ids, scale: float, padding_idx):
        from . import cuda_ops
        ctx.save_for_backward(ids)
        ctx.tref, ctx.scale, ctx.pad = table, scale, padding_idx
        return cuda_ops.embed_fwd(table, ids, scale)

    @staticmethod
    def backward(ctx, dout):
        from . import cuda_ops
        (ids,) = ctx.saved_tensors
        t = ctx.tref
        mg = getattr(t, "main_grad", None)
        if mg is not None:
            cuda_ops.embed_bwd(dout, ids, mg, ctx.scale, ctx.pad)
            _notify(t)
            return None, None, None, None
        g = torch.zeros(t.shape, dtype=torch.float32, device=t.device)
        cuda_ops.embed_bwd(dout, ids, g, ctx.scale, ctx.pad)
        return g.to(t.dtype), None, None, None


def embedding(table, ids, scale: float = 1.0, padding_idx=None):
    return EmbeddingFn.apply(table, ids, scale, padding_idx)


class SeqConcatFn(torch.autograd.Function):
    """``cat([a, c], dim=1)`` with the copy done by one kernel; the gradients are the two slices of the incoming
    gradient (views: nothing is copied in the backward)."""

    @staticmethod
    def forward(ctx, a: Tensor, c: Tensor) -> Tensor:
        from . import cuda_ops
        ctx.s1 = a.shape[1]
        return cuda_ops.seq_concat(a, c)

    @staticmethod
    def backward(ctx, g: Tensor):
        return (g[:, :ctx.s1] if ctx.needs_input_grad[0] else None,
                g[:, ctx.s1:] if ctx.needs_input_grad[1] else None)
