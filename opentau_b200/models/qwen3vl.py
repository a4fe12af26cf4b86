"""Qwen3-VL backbone written on the shared kernels: vision transformer with 2x2 patch merging and deepstack
taps, text decoder with per-head q/k RMS-norm, SwiGLU and interleaved 3-axis MRoPE.

The reference treats the backbone as a stock HuggingFace black box run under ``no_grad`` to obtain per-layer
K/V (OpenTau ``src/opentau/policies/cosmos3/qwen3vl_with_expert.py:540-610``).  Owning it here is what
makes tensor-parallel execution of the frozen 32B backbone possible.  Module names follow the HF layout
(``model.visual.*``, ``model.language_model.*``) so checkpoints load by key.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from .. import ops
from .layers import LayerNorm, Linear, Tower, TowerConfig, _merge_hook, _split_hook


def qwen3_text_config(**over) -> TowerConfig:
    """Qwen3-VL-32B text tower by default."""
    return TowerConfig(**{**dict(hidden_size=5120, num_hidden_layers=64, num_attention_heads=64,
                                 num_key_value_heads=8, head_dim=128, intermediate_size=25600, vocab_size=151936,
                                 hidden_act="silu", rope_theta=5_000_000.0, norm_unit_offset=False, qk_norm=True,
                                 embed_scale=False, mrope_sections=(24, 20, 20)), **over})


@dataclass
class Qwen3VLVisionConfig:
    hidden_size: int = 1152
    depth: int = 27
    num_heads: int = 16
    intermediate_size: int = 4304
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    in_channels: int = 3
    out_hidden_size: int = 5120
    num_position_embeddings: int = 2304
    deepstack_visual_indexes: tuple[int, ...] = (8, 16, 24)
    hidden_act: str = "gelu_tanh"


class _VisionAttention(nn.Module):
    def __init__(self, cfg: Qwen3VLVisionConfig):
        super().__init__()
        d = cfg.hidden_size
        self.h, self.hd = cfg.num_heads, d // cfg.num_heads
        self.qkv = Linear(d, 3 * d, bias=True)
        self.proj = Linear(d, d, bias=True)

    def forward(self, x: Tensor, cos: Tensor, sin: Tensor, residual: Tensor) -> Tensor:
        B, S, d = x.shape
        q, k, v = self.qkv(x).split(d, dim=-1)
        q = ops.rope(q.unflatten(-1, (self.h, self.hd)), cos, sin)
        k = ops.rope(k.unflatten(-1, (self.h, self.hd)), cos, sin)
        o = ops.mha(q, k, v.unflatten(-1, (self.h, self.hd)), self.hd ** -0.5)
        return self.proj(o, residual=residual)


class _VisionMLP(nn.Module):
    def __init__(self, cfg: Qwen3VLVisionConfig):
        super().__init__()
        self.act = cfg.hidden_act
        self.linear_fc1 = Linear(cfg.hidden_size, cfg.intermediate_size, bias=True)
        self.linear_fc2 = Linear(cfg.intermediate_size, cfg.hidden_size, bias=True)

    def forward(self, x: Tensor, residual: Tensor) -> Tensor:
        h = ops.linear_act(x, self.linear_fc1.weight, self.linear_fc1.bias, self.act)
        return self.linear_fc2(h, residual=residual)


class _VisionBlock(nn.Module):
    def __init__(self, cfg: Qwen3VLVisionConfig):
        super().__init__()
        self.norm1 = LayerNorm(cfg.hidden_size)
        self.norm2 = LayerNorm(cfg.hidden_size)
        self.attn = _VisionAttention(cfg)
        self.mlp = _VisionMLP(cfg)

    def forward(self, x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        x = self.attn(self.norm1(x), cos, sin, residual=x)
        return self.mlp(self.norm2(x), residual=x)


class _PatchMerger(nn.Module):
    """LayerNorm then MLP over groups of ``merge^2`` neighbouring patches."""

    def __init__(self, cfg: Qwen3VLVisionConfig, postshuffle_norm: bool = False):
        super().__init__()
        self.m2 = cfg.spatial_merge_size ** 2
        self.postshuffle = postshuffle_norm
        d = cfg.hidden_size
        self.norm = LayerNorm(d * self.m2 if postshuffle_norm else d)
        self.linear_fc1 = Linear(d * self.m2, d * self.m2, bias=True)
        self.linear_fc2 = Linear(d * self.m2, cfg.out_hidden_size, bias=True)

    def forward(self, x: Tensor) -> Tensor:
        B, S, d = x.shape
        if self.postshuffle:
            x = self.norm(x.reshape(B, S // self.m2, d * self.m2))
        else:
            x = self.norm(x).reshape(B, S // self.m2, d * self.m2)
        h = ops.act_fn(self.linear_fc1(x), "gelu")
        return self.linear_fc2(h)


class Qwen3VLVisionModel(nn.Module):
    def __init__(self, cfg: Qwen3VLVisionConfig):
        super().__init__()
        self.cfg = cfg
        k = cfg.in_channels * cfg.temporal_patch_size * cfg.patch_size ** 2
        self.patch_embed = nn.ModuleDict({"proj": Linear(k, cfg.hidden_size, bias=True)})
        self.pos_embed = nn.Embedding(cfg.num_position_embeddings, cfg.hidden_size)
        self.blocks = nn.ModuleList([_VisionBlock(cfg) for _ in range(cfg.depth)])
        self.merger = _PatchMerger(cfg)
        self.deepstack_merger_list = nn.ModuleList(
            [_PatchMerger(cfg, postshuffle_norm=True) for _ in cfg.deepstack_visual_indexes if _ < cfg.depth])

    def _grid_order(self, gh: int, gw: int, device) -> tuple[Tensor, Tensor]:
        """Row/column index of every patch, ordered so that each 2x2 merge group is contiguous."""
        m = self.cfg.spatial_merge_size
        r = torch.arange(gh, device=device).view(gh // m, m, 1, 1).expand(gh // m, m, gw // m, m)
        c = torch.arange(gw, device=device).view(1, 1, gw // m, m).expand(gh // m, m, gw // m, m)
        r = r.permute(0, 2, 1, 3).reshape(-1)
        c = c.permute(0, 2, 1, 3).reshape(-1)
        return r, c

    def forward(self, pixels: Tensor) -> tuple[Tensor, list[Tensor], tuple[int, int]]:
        """``pixels (N, 3, H, W)`` in [-1, 1] -> merged tokens ``(N, gh*gw/4, out)``, deepstack features (same
        shape, one per tap) and the merged grid size."""
        cfg = self.cfg
        N, C, H, W = pixels.shape
        p, m = cfg.patch_size, cfg.spatial_merge_size
        H2, W2 = H // (p * m) * (p * m), W // (p * m) * (p * m)
        pixels = pixels[:, :, :H2, :W2]
        gh, gw = H2 // p, W2 // p
        dtype = self.blocks[0].norm1.weight.dtype
        r, c = self._grid_order(gh, gw, pixels.device)
        patches = pixels.view(N, C, gh, p, gw, p).permute(0, 2, 4, 1, 3, 5)       # (N, gh, gw, C, p, p)
        patches = patches[:, r, c]                                                 # merge-group order
        patches = patches[:, :, :, None].expand(-1, -1, -1, cfg.temporal_patch_size, -1, -1)  # still image x2
        x = self.patch_embed["proj"](patches.reshape(N, gh * gw, -1).to(dtype))
        side = int(math.sqrt(cfg.num_position_embeddings))
        pos = self.pos_embed.weight.view(1, side, side, -1).permute(0, 3, 1, 2).float()
        pos = F.interpolate(pos, size=(gh, gw), mode="bilinear", align_corners=False)[0].permute(1, 2, 0)
        x = x + pos[r, c].to(dtype)[None]
        # 2-D rotary: first half of the rotary dims follows the row index, second half the column index
        hd = cfg.hidden_size // cfg.num_heads
        quarter = hd // 4
        inv = 1.0 / (10000.0 ** (torch.arange(quarter, device=pixels.device, dtype=torch.float32) / quarter))
        ang = torch.cat([r[:, None].float() * inv[None], c[:, None].float() * inv[None]], dim=1)  # (S, hd/2)
        cos, sin = ang.cos()[None].expand(N, -1, -1), ang.sin()[None].expand(N, -1, -1)
        taps: list[Tensor] = []
        idxs = [i for i in cfg.deepstack_visual_indexes if i < cfg.depth]
        for li, blk in enumerate(self.blocks):
            x = blk(x, cos, sin)
            if li in idxs:
                taps.append(self.deepstack_merger_list[idxs.index(li)](x))
        return self.merger(x), taps, (gh // m, gw // m)


class _Qwen3VLInner(nn.Module):
    def __init__(self, text: TowerConfig, vision: Qwen3VLVisionConfig):
        super().__init__()
        self.visual = Qwen3VLVisionModel(vision)
        self.language_model = Tower(text, with_embed=True)


class Qwen3VLBackbone(nn.Module):
    """``model.{visual, language_model}`` (+ tied output head)."""

    def __init__(self, text: TowerConfig, vision: Qwen3VLVisionConfig):
        super().__init__()
        self.text_cfg, self.vision_cfg = text, vision
        self.model = _Qwen3VLInner(text, vision)

    @property
    def language_model(self) -> Tower:
        return self.model.language_model

    def embed_prefix(self, images: list[Tensor], img_masks: list[Tensor], lang_tokens: Tensor, lang_masks: Tensor):
        """Builds ``[camera 0 tokens | camera 1 tokens | ... | text]`` embeddings with 3-axis positions.

        Returns ``(embs, pad, positions (3,B,S), deepstack list of (B,S,d) | None-padded, n_img_tokens)``.
        Image tokens of one camera share the temporal index and carry (row, col) offsets; text tokens use the
        same index on all three axes, continuing after the largest index used so far.
        """
        B = lang_tokens.shape[0]
        device = lang_tokens.device
        dtype = self.language_model.embed_tokens.weight.dtype
        embs, pads, pos_parts, deep = [], [], [], None
        start = 0
        n_img = 0
        if images:
            stacked = torch.stack(images, dim=1).flatten(0, 1)
            tok, taps, (mh, mw) = self.model.visual(stacked)
            per = tok.shape[1]
            tok = tok.view(B, len(images) * per, -1).to(dtype)
            embs.append(tok)
            pads.append(torch.stack(img_masks, dim=1)[:, :, None].expand(B, len(images), per).reshape(B, -1))
            deep = [t.view(B, len(images) * per, -1).to(dtype) for t in taps]
            rr = torch.arange(mh, device=device).repeat_interleave(mw)
            cc = torch.arange(mw, device=device).repeat(mh)
            for _ in images:
                t_idx = torch.full_like(rr, start)
                pos_parts.append(torch.stack([t_idx, start + rr, start + cc]))     # (3, per)
                start += max(mh, mw)
            n_img = len(images) * per
        text = self.language_model.embed_tokens(lang_tokens).to(dtype)
        embs.append(text)
        pads.append(lang_masks.bool())
        L = lang_tokens.shape[1]
        tpos = start + torch.arange(L, device=device)
        pos_parts.append(tpos[None].expand(3, -1))
        pos = torch.cat(pos_parts, dim=1)[:, None, :].expand(3, B, -1)
        return torch.cat(embs, 1), torch.cat(pads, 1), pos, deep, n_img
