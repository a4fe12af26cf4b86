"""SigLIP vision tower (So400m/14 geometry by default) and the multimodal projector.

State-dict keys follow HF ``SiglipVisionModel`` (``vision_model.embeddings.patch_embedding.weight`` …)
so reference checkpoints load unchanged.  The patch embedding and the position table stay fp32 under
every dtype cast (OpenTau ``policies/pi05/paligemma_with_expert.py:454-502``,
``utils/transformers_patch.py:306-348``); the convolution is computed as an unfold + GEMM.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from .. import ops
from .layers import LayerNorm, Linear, _merge_hook, _split_hook


@dataclass
class SiglipConfig:
    hidden_size: int = 1152
    intermediate_size: int = 4304
    num_hidden_layers: int = 27
    num_attention_heads: int = 16
    patch_size: int = 14
    image_size: int = 224
    num_channels: int = 3
    layer_norm_eps: float = 1e-6
    hidden_act: str = "gelu_tanh"

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch_size) ** 2


class PatchEmbedding(nn.Module):
    """Non-overlapping patch convolution + learned position table, both pinned to fp32."""

    def __init__(self, cfg: SiglipConfig):
        super().__init__()
        self.cfg = cfg
        self.patch_embedding = nn.Conv2d(cfg.num_channels, cfg.hidden_size, cfg.patch_size, cfg.patch_size)
        self.position_embedding = nn.Embedding(cfg.num_patches, cfg.hidden_size)

    def _apply(self, fn, recurse=True):
        # Keep the fp32 island: a dtype cast of the whole model must not touch these parameters.
        def keep_fp32(t: Tensor) -> Tensor:
            out = fn(t)
            if out.is_floating_point() and out.dtype != torch.float32:
                out = out.to(torch.float32)
            return out
        return super()._apply(keep_fp32, recurse)

    def interpolated_positions(self, gh: int, gw: int) -> Tensor:
        """The square position grid resampled to ``gh x gw`` for native-resolution inputs: bicubic, half-pixel
        centres (what the reference gets from ``interpolate_pos_encoding=True`` of the stock SigLIP embeddings,
        ``utils/transformers_patch.py:293-300``).  A frozen table on the GPU goes through the resample kernel; a
        trainable one through the differentiable library op."""
        tab = self.position_embedding.weight
        g = int(math.sqrt(tab.shape[0]))
        if (gh, gw) == (g, g):
            return tab
        if tab.is_cuda and not ops.oracle_mode() and not (torch.is_grad_enabled() and tab.requires_grad):
            from ..ops import cuda_ops
            return cuda_ops.pos_resample(tab, gh, gw)
        t = tab.view(1, g, g, -1).permute(0, 3, 1, 2)
        t = F.interpolate(t, size=(gh, gw), mode="bicubic", align_corners=False)
        return t.permute(0, 2, 3, 1).reshape(gh * gw, -1)

    def forward(self, pixels: Tensor, out_dtype: torch.dtype) -> Tensor:
        p = self.cfg.patch_size
        B, C, H, W = pixels.shape
        if H % p or W % p:  # pad to a patch multiple with -1 (black after the [-1,1] scaling)
            pixels = F.pad(pixels, (0, (-W) % p, 0, (-H) % p), value=-1.0)
            H, W = pixels.shape[-2:]
        gh, gw = H // p, W // p
        return ops.patch_embed(pixels, self.patch_embedding.weight, self.patch_embedding.bias,
                               self.interpolated_positions(gh, gw), p, out_dtype)


class SiglipAttention(nn.Module):
    def __init__(self, cfg: SiglipConfig):
        super().__init__()
        d, self.h = cfg.hidden_size, cfg.num_attention_heads
        self.hd = d // self.h
        self.qkv_proj = Linear(d, 3 * d, bias=True)
        self.out_proj = Linear(d, d, bias=True)
        self._register_state_dict_hook(_split_hook("qkv_proj", ["q_proj", "k_proj", "v_proj"], [d, d, d]))
        self._register_load_state_dict_pre_hook(
            _merge_hook("qkv_proj", ["q_proj", "k_proj", "v_proj"]), with_module=False)

    def qkv(self, x: Tensor):
        B, S, d = x.shape
        q, k, v = self.qkv_proj(x).split(d, dim=-1)
        return (q.unflatten(-1, (self.h, self.hd)), k.unflatten(-1, (self.h, self.hd)),
                v.unflatten(-1, (self.h, self.hd)))

    def forward(self, x: Tensor, residual: Tensor | None = None) -> Tensor:
        q, k, v = self.qkv(x)
        o = ops.mha(q, k, v, self.hd ** -0.5)
        return self.out_proj(o, residual=residual)


class SiglipMLP(nn.Module):
    def __init__(self, cfg: SiglipConfig):
        super().__init__()
        self.act = cfg.hidden_act
        self.fc1 = Linear(cfg.hidden_size, cfg.intermediate_size, bias=True)
        self.fc2 = Linear(cfg.intermediate_size, cfg.hidden_size, bias=True)

    def forward(self, x: Tensor, residual: Tensor | None = None) -> Tensor:
        w = self.fc1.weight
        h = ops.linear_act(x.to(w.dtype) if x.dtype != w.dtype else x, w, self.fc1.bias, self.act)
        return self.fc2(h, residual=residual)


class SiglipEncoderLayer(nn.Module):
    def __init__(self, cfg: SiglipConfig):
        super().__init__()
        self.layer_norm1 = LayerNorm(cfg.hidden_size, cfg.layer_norm_eps)
        self.self_attn = SiglipAttention(cfg)
        self.layer_norm2 = LayerNorm(cfg.hidden_size, cfg.layer_norm_eps)
        self.mlp = SiglipMLP(cfg)

    def forward(self, x: Tensor) -> Tensor:
        x = self.self_attn(self.layer_norm1(x), residual=x)
        return self.mlp(self.layer_norm2(x), residual=x)


class SiglipEncoder(nn.Module):
    def __init__(self, cfg: SiglipConfig):
        super().__init__()
        self.layers = nn.ModuleList([SiglipEncoderLayer(cfg) for _ in range(cfg.num_hidden_layers)])


class SiglipVisionTransformer(nn.Module):
    def __init__(self, cfg: SiglipConfig):
        super().__init__()
        self.cfg = cfg
        self.embeddings = PatchEmbedding(cfg)
        self.encoder = SiglipEncoder(cfg)
        self.post_layernorm = LayerNorm(cfg.hidden_size, cfg.layer_norm_eps)

    def forward(self, pixels: Tensor) -> Tensor:
        dtype = self.post_layernorm.weight.dtype
        x = self.embeddings(pixels, dtype)
        for layer in self.encoder.layers:
            x = layer(x)
        return self.post_layernorm(x)


class SiglipVisionModel(nn.Module):
    """``vision_tower`` in HF naming: wraps the transformer under ``vision_model``."""

    def __init__(self, cfg: SiglipConfig):
        super().__init__()
        self.vision_model = SiglipVisionTransformer(cfg)

    def forward(self, pixels: Tensor) -> Tensor:
        return self.vision_model(pixels)


class MultiModalProjector(nn.Module):
    """Linear map from vision width to the text width (PaliGemma; no ``/sqrt(d)`` rescale)."""

    def __init__(self, vision_dim: int, text_dim: int):
        super().__init__()
        self.linear = Linear(vision_dim, text_dim, bias=True)

    def forward(self, x: Tensor) -> Tensor:
        return self.linear(x)


class Gemma3Projector(nn.Module):
    """Gemma-3 projector: average-pool the patch grid to ``tokens_per_image`` tokens, RMSNorm, project."""

    def __init__(self, vision_dim: int, text_dim: int, patches_per_side: int, tokens_per_side: int = 16,
                 eps: float = 1e-6):
        super().__init__()
        from .layers import RMSNorm
        self.mm_input_projection_weight = nn.Parameter(torch.zeros(vision_dim, text_dim))
        nn.init.normal_(self.mm_input_projection_weight, std=0.02)
        self.mm_soft_emb_norm = RMSNorm(vision_dim, eps, unit_offset=True)
        self.patches_per_side, self.tokens_per_side = patches_per_side, tokens_per_side
        self.kernel = patches_per_side // tokens_per_side

    def forward(self, x: Tensor) -> Tensor:
        B, N, C = x.shape
        s = int(math.sqrt(N))
        g = x.transpose(1, 2).reshape(B, C, s, s)
        k = max(1, s // self.tokens_per_side)
        g = F.avg_pool2d(g.float(), kernel_size=k, stride=k).to(x.dtype)
        g = g.flatten(2).transpose(1, 2)
        g = self.mm_soft_emb_norm(g)[0]
        return ops.linear(g, self.mm_input_projection_weight.t().contiguous())
