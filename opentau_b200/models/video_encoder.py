"""SpaceTime SigLIP video encoder: a stock SigLIP tower whose every ``stride``-th layer mixes time.

Behaviour follows OpenTau ``src/opentau/policies/pi07/video_encoder.py:81-778``.  A space-time layer reuses
the layer's own LN1 / QKV / out-proj / MLP weights: one QKV projection of ``LN1(h + PE_t)``; a causal
temporal attention per patch over the ``T`` frames produces mixed values ``V'``; a spatial attention per
frame uses ``(q, k, V')``; the residual is taken on the un-embedded ``h``.  The fixed sinusoidal temporal
embedding has an all-zero row for the current frame, so ``T == 1`` is bit-identical to plain SigLIP.  After
the last layer only the current frame's tokens are normalised and returned.

The temporal attention runs over at most a few frames per (batch, patch) pair — a (T x T) problem — and is
evaluated with the block-causal primitive on a (B*N, T) layout; the spatial attention is the regular
full-attention kernel.
"""

from __future__ import annotations

import math

import torch
from torch import Tensor, nn

from .. import ops
from .siglip import SiglipConfig, SiglipEncoderLayer, SiglipVisionModel


def build_temporal_sinusoidal_pe(num_frames: int, embed_dim: int, min_period: float = 4e-3, max_period: float = 40.0,
                                 dtype=torch.float32, device="cpu") -> Tensor:
    """``(T, embed_dim)`` with row ``T-1`` (the current frame) exactly zero; earlier rows encode the offset into
    the past.  ``max_period`` must exceed the time range to stay alias free."""
    if embed_dim % 2:
        raise ValueError(f"embed_dim ({embed_dim}) must be divisible by 2")
    if num_frames < 1:
        raise ValueError(f"num_frames ({num_frames}) must be >= 1")
    if num_frames - 1 > max_period:
        raise ValueError(f"num_frames ({num_frames}) exceeds the no-alias range of max_period ({max_period}); "
                         f"pass max_period >= {2 * (num_frames - 1)}")
    time = torch.arange(num_frames, dtype=torch.float64, device=device) - (num_frames - 1)
    frac = torch.linspace(0.0, 1.0, embed_dim // 2, dtype=torch.float64, device=device)
    period = min_period * (max_period / min_period) ** frac
    phase = time[:, None] * (2 * math.pi / period)[None, :]
    pe = torch.cat([torch.sin(phase), torch.cos(phase)], dim=-1)
    return (pe - pe[-1:]).to(dtype)


def spacetime_layer_forward(layer: SiglipEncoderLayer, h: Tensor, B: int, T: int, pe: Tensor,
                            frame_valid: Tensor | None = None) -> Tensor:
    """``h ((B*T), N, d)`` -> same shape.  ``frame_valid (B, T)`` marks real (non-padded) history frames."""
    BT, N, d = h.shape
    attn = layer.self_attn
    H, hd = attn.h, attn.hd
    x = h.view(B, T, N, d) + pe[-T:].to(h.dtype).view(1, T, 1, d)
    z = layer.layer_norm1(x.view(BT, N, d))
    q, k, v = attn.qkv(z)                                       # (BT, N, H, hd)
    q5, k5, v5 = (t.reshape(B, T, N, H, hd) for t in (q, k, v))
    # temporal: sequences of T frames per (batch, patch), causal, padded frames invisible
    qt, kt, vt = (t.permute(0, 2, 1, 3, 4).reshape(B * N, T, H, hd) for t in (q5, k5, v5))
    blk = torch.arange(T, dtype=torch.int32, device=h.device)[None].expand(B * N, T)
    if frame_valid is None:
        valid = torch.ones(B * N, T, dtype=torch.bool, device=h.device)
    else:
        valid = frame_valid[:, None, :].expand(B, N, T).reshape(B * N, T)
    v_temp = ops.block_attention(qt.contiguous(), kt.contiguous(), vt.contiguous(), blk, blk, valid, valid,
                                 hd ** -0.5)
    v_mixed = v_temp.view(B, N, T, H, hd).permute(0, 2, 1, 3, 4).reshape(BT, N, H, hd)
    # spatial: per frame over the N patches, values are the temporally mixed ones
    out = ops.mha(q.contiguous(), k.contiguous(), v_mixed.contiguous(), hd ** -0.5)
    h1 = attn.out_proj(out, residual=h)
    return layer.mlp(layer.layer_norm2(h1), residual=h1)


class SpaceTimeSiglipVideoEncoder(nn.Module):
    """Wraps a :class:`SiglipVisionModel`; ``forward(video (B,T,C,H,W))`` returns the current frame's tokens."""

    def __init__(self, vision: SiglipVisionModel, max_num_frames: int = 6, spacetime_layer_stride: int = 4,
                 max_period: float = 40.0):
        super().__init__()
        self.vision = vision
        self.max_num_frames = max_num_frames
        self.stride = spacetime_layer_stride
        d = vision.vision_model.cfg.hidden_size
        self.register_buffer("_temporal_pe", build_temporal_sinusoidal_pe(max_num_frames, d, max_period=max(
            max_period, 2.0 * max(1, max_num_frames - 1))), persistent=False)

    def is_spacetime_layer(self, li: int) -> bool:
        return self.stride > 0 and (li + 1) % self.stride == 0

    def forward(self, video: Tensor, frame_valid: Tensor | None = None, keep_history: bool = False) -> Tensor:
        """``keep_history=False`` (the reference behaviour, ``pi07/video_encoder.py:767-778``): only the current
        frame's tokens ``(B, N, d)`` leave the encoder.  ``keep_history=True`` (long-context variant): every
        frame's tokens, ``(B, T, N, d)``, oldest first."""
        if video.dim() == 4:
            video = video[:, None]
        B, T, C, Hh, Ww = video.shape
        if T > self.max_num_frames:
            raise ValueError(f"{T} frames exceed max_num_frames={self.max_num_frames}")
        if frame_valid is not None:
            # The current (last) frame is always real, also when the history-drop augmentation flags every step as
            # padding (reference tests/policies/test_history_drop_current_frame.py); on a copy: the caller's mask
            # stays as it was.
            frame_valid = frame_valid.bool().clone()
            frame_valid[:, -1] = True
        vm = self.vision.vision_model
        dtype = vm.post_layernorm.weight.dtype
        x = vm.embeddings(video.flatten(0, 1), dtype)            # (B*T, N, d)
        for li, layer in enumerate(vm.encoder.layers):
            if T > 1 and self.is_spacetime_layer(li):
                x = spacetime_layer_forward(layer, x, B, T, self._temporal_pe, frame_valid)
            else:
                x = layer(x)
        if keep_history:
            return vm.post_layernorm(x).view(B, T, *x.shape[1:])
        cur = x.view(B, T, *x.shape[1:])[:, -1]                  # past-frame tokens are dropped here
        return vm.post_layernorm(cur)
