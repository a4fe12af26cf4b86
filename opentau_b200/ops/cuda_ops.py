"""Python side of the sm_100a kernels: argument checks, output allocation, ctypes launches.

Every launcher validates shapes/strides/alignment on the host before the launch (the GPU pool has no
compute-sanitizer), launches on the current torch stream, and returns torch tensors.  A nonzero
return code from the native side raises.  ``check_status()`` reads the device status word that
bounded waits write when they give up.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch
from torch import Tensor

from . import _lib

launch_count = 0  # number of native kernel launches issued through this module (for benchmarks)

EPI_BIAS, EPI_RESIDUAL, EPI_ACCUM, EPI_OUT_F32 = 1, 2, 4, 8
EPI_GLU_GELU, EPI_GLU_SILU, EPI_BIAS_F32, EPI_NO_OUT, EPI_ACT_GELU, EPI_GATE = 16, 32, 64, 128, 256, 512

_status_ptr: dict[int, int] = {}


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: Tensor | None) -> c_void_p:
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"native {what} failed with code {rc}")


def status_pointer() -> int:
    dev = torch.cuda.current_device()
    if dev not in _status_ptr:
        out = c_void_p(0)
        _check(_lib.load("elementwise").otb_status_alloc(ctypes.byref(out)), "status_alloc")
        _status_ptr[dev] = out.value
    return _status_ptr[dev]


def check_status(reset: bool = True) -> None:
    """Raises if any kernel reported a timed-out wait since the last check (synchronises)."""
    dev = torch.cuda.current_device()
    if dev not in _status_ptr:
        return
    torch.cuda.synchronize()
    buf = (ctypes.c_uint * 4)()
    _check(_lib.load("elementwise").otb_status_read(c_void_p(_status_ptr[dev]), buf, int(reset)), "status_read")
    if buf[0] != 0:
        raise RuntimeError(f"kernel wait timed out: kernel={buf[0] >> 16} stage={buf[0] & 0xffff} "
                           f"block={buf[1]} detail={buf[2]} reports={buf[3]}")


# --------------------------------------------------------------------------------------------- GEMM
SKINNY = os.environ.get("OPENTAU_B200_SKINNY_GEMM", "1") != "0"


def use_skinny(layout: str, M: int, N: int, accumulate: bool, bn: int) -> bool:
    """``x @ W^T`` with few rows goes to the weight-streaming split-K kernel."""
    if not SKINNY or layout != "nt" or accumulate or bn:
        return False
    # measured: up to 128 rows the split-K kernel always wins; a 129..256-row product keeps its advantage only while
    # the 128 x 256 tiling has too few tiles (N <= 8192); beyond that the persistent kernel is faster
    return M <= 128 or (M <= 256 and N <= 8192)


def gemm(a: Tensor, b: Tensor, layout: str, bias: Tensor | None = None, residual: Tensor | None = None,
         out: Tensor | None = None, accumulate: bool = False, out_dtype: torch.dtype | None = None,
         glu: str | None = None, glu_out: Tensor | None = None, store_out: bool = True, act: str | None = None,
         bn: int = 0, splits: int = 0, gate: Tensor | None = None) -> Tensor:
    """tcgen05 GEMM.  layout 'nt': a(M,K) b(N,K); 'nn': a(M,K) b(K,N); 'tn': a(K,M) b(K,N).  ``bn`` forces the column
    tile of the persistent kernel, ``splits`` (1, 2, 4, 8) forces the weight-streaming split-K kernel."""
    global launch_count
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "gemm expects bf16 operands"
    if a.stride(-1) != 1 or (a.stride(0) % 8) or (a.data_ptr() % 16):
        a = a.contiguous()
    if b.stride(-1) != 1 or (b.stride(0) % 8) or (b.data_ptr() % 16):
        b = b.contiguous()
    if layout == "nt":
        M, K = a.shape
        N, Kb = b.shape
        a_mn, b_mn = 0, 0
    elif layout == "nn":
        M, K = a.shape
        Kb, N = b.shape
        a_mn, b_mn = 0, 1
    elif layout == "tn":
        K, M = a.shape
        Kb, N = b.shape
        a_mn, b_mn = 1, 1
    else:
        raise ValueError(layout)
    if K != Kb:
        raise ValueError(f"inner dimensions differ: {tuple(a.shape)} x {tuple(b.shape)} ({layout})")
    if N % 8:
        raise ValueError(f"N={N} must be a multiple of 8")
    flags = 0
    odt = out_dtype or (out.dtype if out is not None else torch.bfloat16)
    if out is None and store_out:
        out = torch.empty(M, N, dtype=odt, device=a.device)
    if out is not None:
        if out.shape != (M, N) or out.stride(1) != 1 or out.stride(0) % 8 or out.data_ptr() % 16:
            raise ValueError("bad output tensor for gemm")
        if out.dtype == torch.float32:
            flags |= EPI_OUT_F32
        elif out.dtype != torch.bfloat16:
            raise ValueError("gemm output must be bf16 or fp32")
    else:
        flags |= EPI_NO_OUT
    if accumulate:
        flags |= EPI_ACCUM
    if bias is not None:
        if bias.numel() != N:
            raise ValueError("bias size")
        flags |= EPI_BIAS
        if bias.dtype == torch.float32:
            flags |= EPI_BIAS_F32
        elif bias.dtype != torch.bfloat16:
            raise ValueError("bias dtype")
        bias = bias.contiguous()
    if act == "gelu_tanh":
        flags |= EPI_ACT_GELU
    elif act is not None:
        raise ValueError(act)
    ldr = 0
    if residual is not None:
        if residual.shape != (M, N) or residual.dtype != torch.bfloat16 or residual.stride(1) != 1:
            raise ValueError("bad residual for gemm")
        flags |= EPI_RESIDUAL
        ldr = residual.stride(0)
    ldo2 = 0
    if glu is not None:
        flags |= EPI_GLU_GELU if glu == "gelu_tanh" else EPI_GLU_SILU
        if glu_out is None:
            glu_out = torch.empty(M, N // 2, dtype=torch.bfloat16, device=a.device)
        ldo2 = glu_out.stride(0)
    if splits and (layout != "nt" or accumulate):
        raise ValueError("the split-K kernel computes a @ b^T without accumulation")
    skinny = bool(splits) or use_skinny(layout, M, N, accumulate, bn)
    g_stride, g_rows = 0, 1
    if gate is not None:
        # out = residual + gate * (a @ b^T): rows of N gates, one per `M / gate rows` consecutive output rows
        if not skinny or residual is None or gate.dim() != 2 or gate.shape[1] != N or gate.stride(1) != 1 \
                or gate.dtype != torch.bfloat16 or M % gate.shape[0]:
            raise ValueError("a gated residual epilogue needs the few-row kernel, a residual and (rows, N) bf16 gates")
        flags |= EPI_GATE
        g_stride, g_rows = gate.stride(0), M // gate.shape[0]
    if skinny:
        rc = _lib.load("gemm_skinny_tcgen05").otb_gemm_skinny_bf16(
            _p(a), _p(b), _p(out), c_int(M), c_int(N), c_int(K), c_longlong(a.stride(0)), c_longlong(b.stride(0)),
            c_longlong(out.stride(0) if out is not None else N), _p(bias), _p(residual), c_longlong(ldr), _p(glu_out),
            c_longlong(ldo2), _p(gate), c_longlong(g_stride), c_int(g_rows), c_int(flags), c_int(splits),
            c_void_p(status_pointer()), _stream())
        _check(rc, f"gemm_skinny[{M}x{N}x{K}]")
        launch_count += 1
        if glu is not None:
            return glu_out if not store_out else (out, glu_out)
        return out
    rc = _lib.load("gemm_tcgen05").otb_gemm_bf16(
        _p(a), _p(b), _p(out), c_int(M), c_int(N), c_int(K), c_longlong(a.stride(0)), c_longlong(b.stride(0)),
        c_longlong(out.stride(0) if out is not None else N), c_int(a_mn), c_int(b_mn), _p(bias), _p(residual),
        c_longlong(ldr), _p(glu_out), c_longlong(ldo2), c_int(flags), c_int(bn), c_void_p(status_pointer()),
        _stream())
    _check(rc, f"gemm[{layout} {M}x{N}x{K}]")
    launch_count += 1
    if glu is not None:
        return glu_out if not store_out else (out, glu_out)
    return out


# --------------------------------------------------------------------------------------------- norms
def _rows(x: Tensor) -> tuple[Tensor, int, int]:
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    if x2.stride(1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    return x2, x2.shape[0], H


def rms_fwd(x: Tensor, w: Tensor | None, eps: float, unit_offset: bool):
    global launch_count
    x2, R, H = _rows(x)
    y = torch.empty(R, H, dtype=x.dtype, device=x.device)
    rstd = torch.empty(R, dtype=torch.float32, device=x.device)
    mode = 0 if w is None else (1 if unit_offset else 2)
    wt = w.to(torch.bfloat16).contiguous() if w is not None else None
    _check(_lib.load("elementwise").otb_rms_fwd(_p(x2), c_longlong(x2.stride(0)), _p(wt), c_void_p(0), c_longlong(0),
                                                c_int(1), _p(y), _p(rstd), c_longlong(R), c_int(H), c_float(eps),
                                                c_int(mode), _stream()), "rms_fwd")
    launch_count += 1
    return y.view(x.shape), rstd


def _bwd_blocks(R: int) -> tuple[int, int]:
    rpb = max(1, (R + 591) // 592)
    return rpb, (R + rpb - 1) // rpb


def _dres_rows(dres: Tensor | None, R: int, H: int) -> Tensor | None:
    if dres is None:
        return None
    d = dres.reshape(R, H)
    return d if d.is_contiguous() else d.contiguous()


def rms_bwd(dy: Tensor, x: Tensor, w: Tensor | None, rstd: Tensor, unit_offset: bool, dres: Tensor | None = None):
    """``dres``: a gradient of the same shape as ``x`` that is added to ``dx`` inside the kernel."""
    global launch_count
    x2, R, H = _rows(x)
    dy2, _, _ = _rows(dy)
    if dy2.stride(0) != H:
        dy2 = dy2.contiguous()
    dx = torch.empty(R, H, dtype=x.dtype, device=x.device)
    mode = 0 if w is None else (1 if unit_offset else 2)
    rpb, nb = _bwd_blocks(R)
    partial = torch.empty(nb, H, dtype=torch.float32, device=x.device) if w is not None else None
    wt = w.to(torch.bfloat16).contiguous() if w is not None else None
    lib = _lib.load("elementwise")
    dr = _dres_rows(dres, R, H)
    _check(lib.otb_rms_bwd(_p(dy2), _p(x2), c_longlong(x2.stride(0)), _p(wt), c_void_p(0), c_longlong(0), c_int(1),
                           _p(rstd), _p(dx), _p(partial), c_void_p(0), c_void_p(0), _p(dr), c_longlong(R), c_int(H),
                           c_int(mode), c_int(rpb), _stream()), "rms_bwd")
    launch_count += 1
    dw = None
    if w is not None:
        dw = torch.empty(H, dtype=torch.bfloat16, device=x.device)
        _check(lib.otb_colsum_partials(_p(partial), c_int(nb), c_int(H), _p(dw), c_int(0), _stream()), "colsum")
        launch_count += 1
        dw = dw.to(w.dtype)
    return dx.view(x.shape), dw


def ada_rms_fwd(x: Tensor, mod: Tensor, eps: float):
    global launch_count
    B, S, H = x.shape
    x2, R, _ = _rows(x)
    mod2 = mod.reshape(-1, 3 * H)
    if mod2.stride(1) != 1 or mod2.stride(0) % 8 or mod2.data_ptr() % 16:
        mod2 = mod2.contiguous()
    rows_per_mod = S if mod.dim() == 2 else 1
    y = torch.empty(R, H, dtype=x.dtype, device=x.device)
    rstd = torch.empty(R, dtype=torch.float32, device=x.device)
    _check(_lib.load("elementwise").otb_rms_fwd(_p(x2), c_longlong(x2.stride(0)), c_void_p(0), _p(mod2),
                                                c_longlong(mod2.stride(0)), c_int(rows_per_mod), _p(y), _p(rstd),
                                                c_longlong(R), c_int(H), c_float(eps), c_int(0), _stream()),
           "ada_rms_fwd")
    launch_count += 1
    return y.view(x.shape), rstd


def ada_rms_bwd(dy: Tensor, x: Tensor, mod: Tensor, rstd: Tensor, dres: Tensor | None = None):
    global launch_count
    B, S, H = x.shape
    x2, R, _ = _rows(x)
    dy2 = dy.reshape(R, H).contiguous()
    mod2 = mod.reshape(-1, 3 * H)
    if mod2.stride(1) != 1 or mod2.stride(0) % 8 or mod2.data_ptr() % 16:
        mod2 = mod2.contiguous()
    rows_per_mod = S if mod.dim() == 2 else 1
    dx = torch.empty(R, H, dtype=x.dtype, device=x.device)
    dscale = torch.empty(R, H, dtype=x.dtype, device=x.device)
    dshift = torch.empty(R, H, dtype=x.dtype, device=x.device)
    _check(_lib.load("elementwise").otb_rms_bwd(_p(dy2), _p(x2), c_longlong(x2.stride(0)), c_void_p(0), _p(mod2),
                                                c_longlong(mod2.stride(0)), c_int(rows_per_mod), _p(rstd), _p(dx),
                                                c_void_p(0), _p(dscale), _p(dshift), _p(_dres_rows(dres, R, H)),
                                                c_longlong(R), c_int(H), c_int(0), c_int(1), _stream()), "ada_rms_bwd")
    launch_count += 1
    dscale, dshift = dscale.view(B, S, H), dshift.view(B, S, H)
    if mod.dim() == 2:
        dscale, dshift = dscale.float().sum(1).to(mod.dtype), dshift.float().sum(1).to(mod.dtype)
    return dx.view(x.shape), dscale, dshift


def ln_fwd(x: Tensor, w: Tensor, b: Tensor, eps: float):
    global launch_count
    x2, R, H = _rows(x)
    if x2.stride(0) != H:
        x2 = x2.contiguous()
    y = torch.empty(R, H, dtype=x.dtype, device=x.device)
    mean = torch.empty(R, dtype=torch.float32, device=x.device)
    rstd = torch.empty(R, dtype=torch.float32, device=x.device)
    _check(_lib.load("elementwise").otb_ln_fwd(_p(x2), _p(w.to(torch.bfloat16).contiguous()),
                                               _p(b.to(torch.bfloat16).contiguous()), _p(y), _p(mean), _p(rstd),
                                               c_longlong(R), c_int(H), c_float(eps), _stream()), "ln_fwd")
    launch_count += 1
    return y.view(x.shape), mean, rstd


def ln_bwd(dy: Tensor, x: Tensor, w: Tensor, mean: Tensor, rstd: Tensor):
    """-> ``dx`` (like x), ``dw``, ``db`` (like w).  One kernel for dx and the per-block weight / bias partials, two
    fixed-order column sums."""
    global launch_count
    x2, R, H = _rows(x)
    dy2, _, _ = _rows(dy)
    if x2.stride(0) != H:
        x2 = x2.contiguous()
    if dy2.stride(0) != H:
        dy2 = dy2.contiguous()
    dx = torch.empty(R, H, dtype=x.dtype, device=x.device)
    rpb, nb = _bwd_blocks(R)
    partial = torch.empty(2, nb, H, dtype=torch.float32, device=x.device)
    lib = _lib.load("elementwise")
    _check(lib.otb_ln_bwd(_p(dy2), _p(x2), _p(w.to(torch.bfloat16).contiguous()), _p(mean), _p(rstd), _p(dx),
                          _p(partial[0]), _p(partial[1]), c_longlong(R), c_int(H), c_int(rpb), _stream()), "ln_bwd")
    out = torch.empty(2, H, dtype=torch.bfloat16, device=x.device)
    for k in range(2):
        _check(lib.otb_colsum_partials(_p(partial[k]), c_int(nb), c_int(H), _p(out[k]), c_int(0), _stream()), "colsum")
    launch_count += 3
    return dx.view(x.shape), out[0].to(w.dtype), out[1].to(w.dtype)


# --------------------------------------------------------------------------------------------- GLU / RoPE
_ACT = {"gelu_tanh": 0, "silu": 1}


def glu_fwd(gu: Tensor, act: str) -> Tensor:
    global launch_count
    gu2, M, I2 = _rows(gu)
    if gu2.stride(0) != I2:
        gu2 = gu2.contiguous()
    h = torch.empty(M, I2 // 2, dtype=gu.dtype, device=gu.device)
    _check(_lib.load("elementwise").otb_glu_fwd(_p(gu2), _p(h), c_longlong(M), c_int(I2 // 2), c_int(_ACT[act]),
                                                _stream()), "glu_fwd")
    launch_count += 1
    return h.view(*gu.shape[:-1], I2 // 2)


def glu_bwd(gu: Tensor, dh: Tensor, act: str, inplace: bool = False) -> Tensor:
    global launch_count
    gu2, M, I2 = _rows(gu)
    if gu2.stride(0) != I2:
        gu2 = gu2.contiguous()
    dh2 = dh.reshape(M, I2 // 2).contiguous()
    dgu = gu2 if inplace else torch.empty_like(gu2)
    _check(_lib.load("elementwise").otb_glu_bwd(_p(gu2), _p(dh2), _p(dgu), c_longlong(M), c_int(I2 // 2),
                                                c_int(_ACT[act]), _stream()), "glu_bwd")
    launch_count += 1
    return dgu.view(gu.shape)


def rope_fwd(x: Tensor, cos: Tensor, sin: Tensor, inverse: bool = False) -> Tensor:
    global launch_count
    B, S, H, D = x.shape
    if x.stride(3) != 1 or any(s % 8 for s in x.stride()[:3]) or x.data_ptr() % 16:
        x = x.contiguous()
    cos = cos.float().contiguous()
    sin = sin.float().contiguous()
    if cos.shape != (B, S, D // 2):
        cos = cos.expand(B, S, D // 2).contiguous()
        sin = sin.expand(B, S, D // 2).contiguous()
    y = torch.empty(B, S, H, D, dtype=x.dtype, device=x.device)
    _check(_lib.load("elementwise").otb_rope(_p(x), c_longlong(x.stride(0)), c_longlong(x.stride(1)),
                                             c_longlong(x.stride(2)), _p(cos), _p(sin), _p(y), c_int(B), c_int(S),
                                             c_int(H), c_int(D), c_int(int(inverse)), _stream()), "rope")
    launch_count += 1
    return y


# --------------------------------------------------------------------------------------------- CE
CE_VOCAB_TILE = 16384      # vocabulary columns per pass of the tiled cross-entropy head


def _ce_tiles(V: int):
    return [(c0, min(V, c0 + CE_VOCAB_TILE)) for c0 in range(0, V, CE_VOCAB_TILE)]


def linear_ce_fwd(h: Tensor, w: Tensor, bias: Tensor | None, labels: Tensor):
    """Per-row cross entropy of ``h @ w.T + b`` and the fp32 log-sum-exp, one vocabulary tile at a time: the logits
    of a tile (rows x <= 16384, fp32) live only until the tile has been folded into the rows' running max / sum,
    so the 257 152-wide language-model head never needs its 8 GB of logits."""
    global launch_count
    R, V = h.shape[0], w.shape[0]
    labels = labels.contiguous()
    lib = _lib.load("elementwise")
    if V <= CE_VOCAB_TILE:
        logits = gemm(h, w, "nt", bias=bias, out_dtype=torch.float32)
        loss = torch.empty(R, dtype=torch.float32, device=h.device)
        lse = torch.empty(R, dtype=torch.float32, device=h.device)
        _check(lib.otb_ce_fwd(_p(logits), _p(labels), _p(loss), _p(lse), c_longlong(R), c_int(V), _stream()), "ce_fwd")
        launch_count += 1
        return loss, lse
    m = torch.full((R,), float("-inf"), dtype=torch.float32, device=h.device)
    s = torch.zeros(R, dtype=torch.float32, device=h.device)
    tgt = torch.zeros(R, dtype=torch.float32, device=h.device)
    tile_lib = _lib.load("train_elementwise")
    for c0, c1 in _ce_tiles(V):
        logits = gemm(h, w[c0:c1], "nt", bias=bias[c0:c1] if bias is not None else None, out_dtype=torch.float32)
        _check(tile_lib.otb_ce_tile_fwd(_p(logits), _p(labels), c_longlong(c0), c_longlong(R), c_int(c1 - c0), _p(m),
                                        _p(s), _p(tgt), _stream()), "ce_tile_fwd")
        launch_count += 1
        del logits
    lse = m + torch.log(s)
    return lse - tgt, lse


def linear_ce_bwd(dloss: Tensor, h: Tensor, w: Tensor, bias: Tensor | None, labels: Tensor, lse: Tensor,
                  dw_into: Tensor | None = None):
    """``(dh, dw, dbias)`` of :func:`linear_ce_fwd`, tile by tile: each tile's logits are recomputed, turned into
    ``(softmax - onehot) * dloss`` (bf16) and consumed by the two gradient products before the next tile starts.
    ``dw_into``: a ``(V, H)`` gradient buffer the weight gradient is ACCUMULATED into (then ``dw`` is None)."""
    global launch_count
    R, V = h.shape[0], w.shape[0]
    lib = _lib.load("elementwise")
    labels = labels.contiguous()
    dl32 = dloss.float().contiguous()
    tiles = _ce_tiles(V)
    dh32 = None
    dw = None if dw_into is not None else torch.empty_like(w)
    db = torch.empty(V, dtype=bias.dtype, device=h.device) if bias is not None else None
    for c0, c1 in tiles:
        wc = w[c0:c1]
        logits = gemm(h, wc, "nt", bias=bias[c0:c1] if bias is not None else None, out_dtype=torch.float32)
        dlogits = torch.empty(R, c1 - c0, dtype=torch.bfloat16, device=h.device)
        lab = labels if c0 == 0 else labels - c0          # a label outside the tile matches no column
        _check(lib.otb_ce_bwd(_p(logits), _p(lab), _p(lse), _p(dl32), _p(dlogits), c_longlong(R), c_int(c1 - c0),
                              _stream()), "ce_bwd")
        launch_count += 1
        del logits
        if len(tiles) == 1:
            dh = gemm(dlogits, wc, "nn")
        else:
            part = gemm(dlogits, wc, "nn", out_dtype=torch.float32)
            dh32 = part if dh32 is None else dh32.add_(part)
        if dw_into is not None:
            gemm(dlogits, h, "tn", out=dw_into[c0:c1], accumulate=True)
        else:
            gemm(dlogits, h, "tn", out=dw[c0:c1])
        if db is not None:
            db[c0:c1] = col_sum(dlogits).to(bias.dtype)
    if len(tiles) > 1:
        dh = dh32.to(h.dtype)
    return dh, dw, db


def col_sum(a: Tensor) -> Tensor:
    global launch_count
    a2, R, H = _rows(a)
    rpb = max(1, (R + 255) // 256)
    nb = (R + rpb - 1) // rpb
    partial = torch.empty(nb, H, dtype=torch.float32, device=a.device)
    lib = _lib.load("elementwise")
    _check(lib.otb_colsum_bf16(_p(a2), c_longlong(R), c_int(H), c_longlong(a2.stride(0)), _p(partial), c_int(rpb),
                               _stream()), "colsum_bf16")
    out = torch.empty(H, dtype=torch.bfloat16, device=a.device)
    _check(lib.otb_colsum_partials(_p(partial), c_int(nb), c_int(H), _p(out), c_int(0), _stream()), "colsum")
    launch_count += 2
    return out


# --------------------------------------------------------------------------------------------- optimizer
def sumsq_partials(g: Tensor, partial: Tensor) -> None:
    global launch_count
    _check(_lib.load("elementwise").otb_sumsq(_p(g), c_longlong(g.numel()), c_int(int(g.dtype == torch.bfloat16)),
                                              _p(partial), c_int(partial.numel()), _stream()), "sumsq")
    launch_count += 1


def clip_coef(partial: Tensor, grad_scale: float, max_norm: float, out: Tensor) -> None:
    global launch_count
    _check(_lib.load("elementwise").otb_clip_coef(_p(partial), c_int(partial.numel()), c_float(grad_scale),
                                                  c_float(max_norm), _p(out), _stream()), "clip_coef")
    launch_count += 1


def adamw(p32: Tensor, g: Tensor, m: Tensor, v: Tensor, p16: Tensor | None, *, lr: float, beta1: float, beta2: float,
          eps: float, weight_decay: float, step: int, scale: Tensor | None = None) -> None:
    global launch_count
    n = p32.numel()
    assert g.numel() == n and m.numel() == n and v.numel() == n
    _check(_lib.load("elementwise").otb_adamw(_p(p32), _p(g), c_int(int(g.dtype == torch.bfloat16)), _p(m), _p(v),
                                              _p(p16), c_longlong(n), c_float(lr), c_float(beta1), c_float(beta2),
                                              c_float(eps), c_float(weight_decay), c_float(1.0 - beta1 ** step),
                                              c_float(1.0 - beta2 ** step), _p(scale), _stream()), "adamw")
    launch_count += 1


# --------------------------------------------------------------------------------------------- images
def resize_with_pad(img: Tensor, width: int, height: int, pad_value: float = -1.0) -> Tensor:
    global launch_count
    N, C, Hin, Win = img.shape
    ratio = max(Win / width, Hin / height)
    rh, rw = int(Hin / ratio), int(Win / ratio)
    x = img.float().contiguous()
    out = torch.empty(N, C, height, width, dtype=torch.float32, device=img.device)
    _check(_lib.load("elementwise").otb_resize_pad(_p(x), _p(out), c_int(N * C), c_int(Hin), c_int(Win), c_int(height),
                                                   c_int(width), c_int(rh), c_int(rw), c_float(pad_value), _stream()),
           "resize_pad")
    launch_count += 1
    return out


def gated_residual(x: Tensor, y: Tensor, gate: Tensor) -> Tensor:
    global launch_count
    B, S, H = x.shape
    x2, y2 = x.reshape(-1, H).contiguous(), y.reshape(-1, H).contiguous()
    g2 = gate.reshape(-1, H) if gate.stride(-1) == 1 else gate.reshape(-1, H).contiguous()
    if g2.stride(0) % 8 or g2.data_ptr() % 16:
        g2 = g2.contiguous()
    rows_per_gate = (B * S) // g2.shape[0]
    out = torch.empty_like(x2)
    _check(_lib.load("elementwise").otb_gated_residual(_p(x2), _p(y2), _p(g2), c_longlong(g2.stride(0)),
                                                       c_int(rows_per_gate), _p(out), c_longlong(B * S), c_int(H),
                                                       _stream()), "gated_residual")
    launch_count += 1
    return out.view(x.shape)


def qkv_post(qkv: Tensor, H: int, Hkv: int, D: int, q_norm, k_norm, cos: Tensor, sin: Tensor,
             k_dst: Tensor | None = None, v_dst: Tensor | None = None):
    global launch_count
    B, T, W = qkv.shape
    assert W == (H + 2 * Hkv) * D and qkv.dtype == torch.bfloat16
    if qkv.stride(-1) != 1 or qkv.stride(0) != T * qkv.stride(1):
        qkv = qkv.contiguous()
    cos = cos.float().contiguous()
    sin = sin.float().contiguous()
    if cos.shape != (B, T, D // 2):
        cos = cos.expand(B, T, D // 2).contiguous()
        sin = sin.expand(B, T, D // 2).contiguous()
    q = torch.empty(B, T, H, D, dtype=qkv.dtype, device=qkv.device)
    if k_dst is None:
        k_dst = torch.empty(B, T, Hkv, D, dtype=qkv.dtype, device=qkv.device)
        v_dst = torch.empty(B, T, Hkv, D, dtype=qkv.dtype, device=qkv.device)
    for t in (k_dst, v_dst):
        if t.shape != (B, T, Hkv, D) or t.stride(3) != 1 or t.stride(2) != D or t.dtype != qkv.dtype:
            raise ValueError("k / v destination must be (B,T,Hkv,D) with dense heads")
    norm = q_norm is not None
    qw = q_norm.weight.to(qkv.dtype) if norm else None
    kw = k_norm.weight.to(qkv.dtype) if norm else None
    _check(_lib.load("elementwise").otb_qkv_post(
        _p(qkv), c_longlong(qkv.stride(1)), _p(qw), _p(kw), c_float(q_norm.eps if norm else 0.0),
        c_int(int(q_norm.unit_offset) if norm else 0), _p(cos), _p(sin), _p(q), _p(k_dst), c_longlong(k_dst.stride(0)),
        c_longlong(k_dst.stride(1)), _p(v_dst), c_longlong(v_dst.stride(0)), c_longlong(v_dst.stride(1)), c_int(B),
        c_int(T), c_int(H), c_int(Hkv), c_int(D), _stream()), "qkv_post")
    launch_count += 1
    return q, k_dst, v_dst


def patch_embed(pixels: Tensor, weight: Tensor, bias: Tensor, pos: Tensor, patch: int, out_dtype: torch.dtype) -> Tensor:
    """``pixels (B,C,H,W)`` fp32 / bf16, ``weight (N, C*p*p)``, ``bias (N)``, ``pos (gh*gw, N)`` all fp32 ->
    ``(B, gh*gw, N)`` in ``out_dtype``."""
    global launch_count
    B, C, H, W = pixels.shape
    N = weight.shape[0]
    if pixels.dtype not in (torch.float32, torch.bfloat16):
        pixels = pixels.float()
    pixels = pixels.contiguous()
    weight, bias, pos = weight.float().contiguous(), bias.float().contiguous(), pos.float().contiguous()
    out = torch.empty(B, (H // patch) * (W // patch), N, dtype=out_dtype, device=pixels.device)
    _check(_lib.load("elementwise").otb_patch_embed(
        _p(pixels), c_int(int(pixels.dtype == torch.bfloat16)), _p(weight), _p(bias), _p(pos), _p(out),
        c_int(int(out_dtype == torch.bfloat16)), c_int(B), c_int(C), c_int(H), c_int(W), c_int(patch), c_int(N),
        _stream()), "patch_embed")
    launch_count += 1
    return out


def time_embed(time: Tensor, dim: int, min_period: float, max_period: float, out_dtype: torch.dtype) -> Tensor:
    global launch_count
    t = time.float().contiguous()
    out = torch.empty(*t.shape, dim, dtype=out_dtype, device=t.device)
    _check(_lib.load("elementwise").otb_time_embed(_p(t), _p(out), c_longlong(t.numel()), c_int(dim),
                                                   c_float(min_period), c_float(max_period),
                                                   c_int(int(out_dtype == torch.bfloat16)), _stream()), "time_embed")
    launch_count += 1
    return out


def euler_step_(x: Tensor, v: Tensor, dt: float, frozen: Tensor | None = None, prefix: Tensor | None = None) -> Tensor:
    """In place: ``x += dt * v``; rows with ``frozen`` set take ``prefix`` instead.  ``x`` fp32 contiguous (B,T,D)."""
    global launch_count
    assert x.dtype == torch.float32 and x.is_contiguous() and v.shape == x.shape
    v = v.contiguous()
    fz = pf = None
    if frozen is not None and prefix is not None:
        fz = frozen.contiguous()
        fz = fz.view(torch.uint8) if fz.dtype == torch.bool else fz.to(torch.uint8)
        pf = prefix.float().contiguous()
    D = x.shape[-1]
    _check(_lib.load("elementwise").otb_euler_step(_p(x), _p(v), c_int(int(v.dtype == torch.bfloat16)), c_float(dt),
                                                   _p(fz), _p(pf), c_longlong(x.numel() // D), c_int(D), _stream()),
           "euler_step")
    launch_count += 1
    return x


def flow_interpolate(actions: Tensor, noise: Tensor, time: Tensor) -> tuple[Tensor, Tensor]:
    global launch_count
    a, n, t = actions.float().contiguous(), noise.float().contiguous(), time.float().contiguous()
    x_t, u_t = torch.empty_like(a), torch.empty_like(a)
    D = a.shape[-1]
    _check(_lib.load("elementwise").otb_flow_interpolate(_p(a), _p(n), _p(t), _p(x_t), _p(u_t),
                                                         c_longlong(a.numel() // D), c_int(D), _stream()),
           "flow_interpolate")
    launch_count += 1
    return x_t, u_t


# --------------------------------------------------------------------------------------------- attention
def attn_fwd(q, k, v, q_blk, k_blk, q_valid, k_valid, scale):
    from . import attention
    return attention.attn_fwd(q, k, v, q_blk, k_blk, q_valid, k_valid, scale)


def attn_bwd(do, q, k, v, o, lse, q_blk, k_blk, q_valid, k_valid, scale):
    from . import attention
    return attention.attn_bwd(do, q, k, v, o, lse, q_blk, k_blk, q_valid, k_valid, scale)


# --------------------------------------------------------------------------------------------- training elementwise
def dropout_residual_fwd(x: Tensor, y: Tensor, gate: Tensor | None, p: float, seed: int) -> Tensor:
    """``x + gate * dropout(y, p)`` for ``(B, T, H)`` bf16 tensors (``gate (B, 1 | T, H)`` or None), one pass; the keep
    mask comes from ``seed`` and is never stored."""
    global launch_count
    H = x.shape[-1]
    x2, y2 = x.reshape(-1, H), y.reshape(-1, H)
    x2 = x2 if x2.is_contiguous() else x2.contiguous()
    y2 = y2 if y2.is_contiguous() else y2.contiguous()
    rows = x2.shape[0]
    g2, stride, rpg = None, 0, 1
    if gate is not None:
        g2 = gate.reshape(-1, H)
        if g2.stride(1) != 1 or g2.stride(0) % 8 or g2.data_ptr() % 16:
            g2 = g2.contiguous()
        stride, rpg = g2.stride(0), rows // g2.shape[0]
    out = torch.empty_like(x2)
    _check(_lib.load("train_elementwise").otb_drop_res_fwd(
        _p(x2), _p(y2), _p(g2), c_longlong(stride), c_int(rpg), _p(out), c_longlong(rows), c_int(H), c_float(p),
        ctypes.c_ulonglong(seed), _stream()), "drop_res_fwd")
    launch_count += 1
    return out.view(x.shape)


def dropout_residual_bwd(dout: Tensor, y: Tensor | None, gate: Tensor | None, p: float, seed: int):
    """Gradients of :func:`dropout_residual_fwd` w.r.t. ``y`` (and ``gate``, as fp32 ``(gate rows, H)``)."""
    global launch_count
    H = dout.shape[-1]
    d2 = dout.reshape(-1, H)
    d2 = d2 if d2.is_contiguous() else d2.contiguous()
    rows = d2.shape[0]
    g2, stride, rpg, dgate, y2 = None, 0, 1, None, None
    if gate is not None:
        g2 = gate.reshape(-1, H)
        if g2.stride(1) != 1 or g2.stride(0) % 8 or g2.data_ptr() % 16:
            g2 = g2.contiguous()
        stride, rpg = g2.stride(0), rows // g2.shape[0]
        dgate = torch.empty(g2.shape[0], H, dtype=torch.float32, device=dout.device)
        y2 = y.reshape(-1, H)
        y2 = y2 if y2.is_contiguous() else y2.contiguous()
    dy = torch.empty_like(d2)
    _check(_lib.load("train_elementwise").otb_drop_res_bwd(
        _p(d2), _p(y2), _p(g2), c_longlong(stride), c_int(rpg), _p(dy), _p(dgate), c_longlong(rows), c_int(H),
        c_float(p), ctypes.c_ulonglong(seed), _stream()), "drop_res_bwd")
    launch_count += 1
    return dy.view(dout.shape), dgate


def masked_mse_fwd(u: Tensor, v: Tensor, frozen: Tensor | None, pad: Tensor | None, real_dim: Tensor | None):
    """Per-sample ``(sum of squared differences, number of counted elements)`` of ``(B, T, D)`` fp32 tensors."""
    global launch_count
    B, T, D = u.shape
    sums = torch.empty(B, dtype=torch.float32, device=u.device)
    counts = torch.empty(B, dtype=torch.float32, device=u.device)
    _check(_lib.load("train_elementwise").otb_masked_mse_fwd(_p(u), _p(v), _p(frozen), _p(pad), _p(real_dim), c_int(B),
                                                             c_int(T), c_int(D), _p(sums), _p(counts), _stream()),
           "masked_mse_fwd")
    launch_count += 1
    return sums, counts


def masked_mse_bwd(u: Tensor, v: Tensor, frozen: Tensor | None, pad: Tensor | None, real_dim: Tensor | None,
                   coef: Tensor) -> Tensor:
    global launch_count
    B, T, D = u.shape
    dv = torch.empty_like(v)
    _check(_lib.load("train_elementwise").otb_masked_mse_bwd(_p(u), _p(v), _p(frozen), _p(pad), _p(real_dim), c_int(B),
                                                             c_int(T), c_int(D), _p(coef), _p(dv), _stream()),
           "masked_mse_bwd")
    launch_count += 1
    return dv


def embed_fwd(table: Tensor, ids: Tensor, scale: float) -> Tensor:
    global launch_count
    H = table.shape[1]
    flat = ids.reshape(-1).to(torch.int64).contiguous()
    out = torch.empty(flat.numel(), H, dtype=table.dtype, device=table.device)
    _check(_lib.load("train_elementwise").otb_embed_fwd(_p(table), _p(flat), _p(out), c_longlong(flat.numel()), c_int(H),
                                                        c_longlong(table.shape[0]), c_float(scale), _stream()),
           "embed_fwd")
    launch_count += 1
    return out.view(*ids.shape, H)


def embed_bwd(dout: Tensor, ids: Tensor, grad: Tensor, scale: float, padding_idx: int | None = None) -> None:
    """``grad[ids[i], :] += scale * dout[i, :]`` for a ``(V, H)`` bf16 or fp32 gradient table, deterministic (rows
    with the same id are summed in token order by one warp)."""
    global launch_count
    H = grad.shape[1]
    flat = ids.reshape(-1).to(torch.int64)
    sorted_ids, order = torch.sort(flat, stable=True)
    n = flat.numel()
    if n == 0:
        return
    d2 = dout.reshape(-1, H)
    d2 = d2 if d2.is_contiguous() else d2.contiguous()
    _check(_lib.load("train_elementwise").otb_embed_bwd(
        _p(d2), _p(sorted_ids), _p(order), c_longlong(n), _p(grad), c_int(int(grad.dtype == torch.float32)), c_int(H),
        c_longlong(grad.shape[0]), c_longlong(-1 if padding_idx is None else padding_idx), c_float(scale), _stream()),
        "embed_bwd")
    launch_count += 1


def pos_resample(table: Tensor, gh: int, gw: int) -> Tensor:
    """Bicubic resample of a square ``(g*g, d)`` fp32 position table to ``(gh*gw, d)``."""
    global launch_count
    import math
    g = int(math.isqrt(table.shape[0]))
    tab = table.detach().float().contiguous()
    out = torch.empty(gh * gw, tab.shape[1], dtype=torch.float32, device=tab.device)
    _check(_lib.load("train_elementwise").otb_pos_resample(_p(tab), c_int(g), c_int(tab.shape[1]), _p(out), c_int(gh),
                                                           c_int(gw), _stream()), "pos_resample")
    launch_count += 1
    return out


def seq_concat(a: Tensor, c: Tensor) -> Tensor:
    """``cat([a, c], dim=1)`` for bf16 ``(B, S, ...)`` tensors whose trailing dims are dense: one vectorised copy kernel
    (the library's batched concatenation moves these shapes at a tenth of the copy bandwidth)."""
    global launch_count
    B, S1, S2 = a.shape[0], a.shape[1], c.shape[1]
    E = a[0, 0].numel() if S1 else c[0, 0].numel()
    out = torch.empty(B, S1 + S2, *a.shape[2:], dtype=a.dtype, device=a.device)
    _check(_lib.load("train_elementwise").otb_seq_concat(
        _p(a), c_longlong(a.stride(0)), c_longlong(a.stride(1)), _p(c), c_longlong(c.stride(0)), c_longlong(c.stride(1)),
        _p(out), c_longlong(B), c_int(S1), c_int(S2), c_int(E), _stream()), "seq_concat")
    launch_count += 1
    return out


def zero_(t: Tensor) -> Tensor:
    """``t.zero_()`` for a dense CUDA tensor through the driver's memset (about twice the rate of the element-wise fill
    on multi-GB buffers); anything else falls back to ``t.zero_()``."""
    global launch_count
    if not (t.is_cuda and t.is_contiguous() and t.numel() > 0):
        return t.zero_()
    from ctypes import c_ulonglong
    _check(_lib.load("train_elementwise").otb_zero_bytes(_p(t), c_ulonglong(t.numel() * t.element_size()), _stream()),
           "zero_bytes")
    launch_count += 1
    return t


def seq_concat_supported(a: Tensor, c: Tensor) -> bool:
    if not (a.is_cuda and a.dtype == c.dtype == torch.bfloat16 and a.dim() == c.dim() >= 3):
        return False
    if a.shape[0] != c.shape[0] or a.shape[2:] != c.shape[2:] or a.shape[1] == 0 or c.shape[1] == 0:
        return False
    E = a[0, 0].numel()

    def rows_dense(t: Tensor) -> bool:
        exp = 1
        for size, stride in zip(reversed(t.shape[2:]), reversed(t.stride()[2:])):
            if size != 1 and stride != exp:
                return False
            exp *= size
        return t.stride(0) % 8 == 0 and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0
    return E % 8 == 0 and rows_dense(a) and rows_dense(c)
