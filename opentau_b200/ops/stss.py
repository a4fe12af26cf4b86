"""Local space-time correlation (the STSS transformation of the motion module) as one kernel each way.

``local_window_correlation(x, T, H, W, L, k)`` takes the token-major feature matrix ``x (B, T, H*W, C)`` (already
normalised for the cosine variant) and returns ``(B, T, H*W, L, k*k)``: inner products with the features inside the
``(L, k, k)`` window, zeros outside the image.  On CUDA bf16 / fp32 tensors it runs ``csrc/stss_corr.cu``; elsewhere a
PyTorch body that gathers the window with ``unfold`` (reference math:
``src/opentau/policies/pi05_mem/motion_module.py:84-200``).
"""

from __future__ import annotations

from ctypes import c_int, c_void_p

import torch
import torch.nn.functional as F
from torch import Tensor


def target_frames(T: int, L: int, device) -> Tensor:
    """``(T, L)`` index of the frame that offset ``l`` of frame ``t`` looks at (ends clamped; ``L == 1``: the previous
    frame)."""
    if L > 1:
        pad = L // 2
        return (torch.arange(T, device=device)[:, None] + torch.arange(-pad, pad + 1, device=device)[None, :]).clamp(0, T - 1)
    return (torch.arange(T, device=device) - 1).clamp(min=0)[:, None]


def dense_window_correlation(x: Tensor, T: int, H: int, W: int, L: int, k: int) -> Tensor:
    B, _, HW, C = x.shape
    v = x.view(B, T, H, W, C).permute(0, 1, 4, 2, 3)                               # (B, T, C, H, W)
    idx = target_frames(T, L, x.device)
    tgt = v[:, idx].reshape(-1, C, H, W)                                          # (B*T*L, C, H, W)
    src = v[:, :, None].expand(B, T, idx.shape[1], C, H, W).reshape(-1, C, H, W)
    win = F.unfold(tgt, kernel_size=k, padding=k // 2).view(-1, C, k * k, H, W)
    corr = torch.einsum("nchw,nckhw->nhwk", src, win)                             # (B*T*L, H, W, k*k)
    return corr.view(B, T, idx.shape[1], HW, k * k).permute(0, 1, 3, 2, 4).contiguous()


def native_supported(x: Tensor) -> bool:
    if not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float32):
        return False
    per = 16 // x.element_size()
    return x.shape[-1] % per == 0 and x.shape[-1] // per <= 256


def _launch(name: str, *args) -> None:
    from . import _lib, cuda_ops
    rc = getattr(_lib.load("stss_corr"), name)(*args, cuda_ops._stream())
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}")
    cuda_ops.launch_count += 1


class _WindowCorrelation(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, T: int, H: int, W: int, L: int, k: int) -> Tensor:
        x = x.contiguous()
        B, _, HW, C = x.shape
        out = torch.empty(B, T, HW, L, k * k, dtype=x.dtype, device=x.device)
        _launch("otb_stss_corr_fwd", c_void_p(x.data_ptr()), c_void_p(out.data_ptr()), c_int(B), c_int(T), c_int(H),
                c_int(W), c_int(C), c_int(L), c_int(k), c_int(x.element_size()))
        ctx.save_for_backward(x)
        ctx.geom = (T, H, W, L, k)
        return out

    @staticmethod
    def backward(ctx, g: Tensor):
        (x,) = ctx.saved_tensors
        T, H, W, L, k = ctx.geom
        B, _, HW, C = x.shape
        g = g.contiguous().to(x.dtype)
        dx = torch.empty_like(x)
        _launch("otb_stss_corr_bwd", c_void_p(x.data_ptr()), c_void_p(g.data_ptr()), c_void_p(dx.data_ptr()), c_int(B),
                c_int(T), c_int(H), c_int(W), c_int(C), c_int(L), c_int(k), c_int(x.element_size()))
        return dx, None, None, None, None, None


def local_window_correlation(x: Tensor, T: int, H: int, W: int, L: int, k: int) -> Tensor:
    from . import oracle_mode
    if x.shape[1] != T or x.shape[2] != H * W:
        raise ValueError(f"expected (B, {T}, {H * W}, C), got {tuple(x.shape)}")
    if L % 2 == 0 or k % 2 == 0:
        raise ValueError(f"window sizes must be odd, got L={L} k={k}")
    if native_supported(x) and not oracle_mode():
        return _WindowCorrelation.apply(x, T, H, W, L, k)
    return dense_window_correlation(x, T, H, W, L, k)
