"""Space-Time Self-Similarity (STSS) motion module and the SigLIP video encoder that hosts it.

What it computes (reference ``src/opentau/policies/pi05_mem/motion_module.py:84-458`` and
``pi05_mem/rldx_video_encoder.py:63-282``): every patch feature of every frame is correlated (cosine by default)
with the features inside a ``(L, k, k)`` space-time window around it — ``L`` neighbouring frames with the ends
clamped, a ``k x k`` patch neighbourhood with zeros outside the image — the ``k*k`` similarities become channels,
two pointwise convolutions (with a per-sample GroupNorm) mix similarities and then the ``L`` frame offsets, and a
zero-initialised projection turns the result into a residual on the vision features:
``v'(t) = v(t) + S(STSS(v(t)))``.

The local window is read directly instead of forming the global ``(HW x HW)`` correlation and slicing diagonals out of
it: ``O(HW k^2 C)`` work instead of ``O((HW)^2 C)``; on the GPU one kernel each way computes the similarities from
the token-major features without materialising the window (``ops/csrc/stss_corr.cu``).  All convolutions of the default ``lite`` integration are 1x1x1, i.e. per-token linear maps, and run
as GEMMs; parameter names and shapes match the reference (``stss_encoders.N.stss_extraction.conv0.0.weight``
``(C, k*k, 1, 1, 1)`` ...) so checkpoints interchange.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from .siglip import SiglipVisionModel


def _make_norm3d(c: int, kind: str) -> nn.Module:
    if kind == "groupnorm":
        return nn.GroupNorm(1, c)
    if kind == "batchnorm":
        return nn.BatchNorm3d(c)
    if kind == "syncbn":
        return nn.SyncBatchNorm(c)
    raise ValueError(f"unknown norm {kind!r}")


def local_correlation(src: Tensor, tgt: Tensor, k: int, corr_func: str = "cosine") -> Tensor:
    """``src, tgt (N, C, H, W)`` -> ``(N, H, W, k, k)`` with ``out[n,h,w,u,v] = <src[n,:,h,w], tgt[n,:,h+u-k//2, w+v-k//2]>``
    (0 outside the image; ``-inf`` before the softmax variant)."""
    N, C, H, W = src.shape
    if corr_func == "cosine":
        src, tgt = F.normalize(src, p=2, dim=1), F.normalize(tgt, p=2, dim=1)
    elif corr_func in ("dotproduct", "dotproduct_softmax"):
        src = src * C ** -0.5
    else:
        raise ValueError(f"unknown corr_func {corr_func!r}")
    d = k // 2
    win = F.unfold(tgt, kernel_size=k, padding=d).view(N, C, k * k, H, W)       # zero padded neighbourhoods
    corr = torch.einsum("nchw,nckhw->nhwk", src, win)
    if corr_func == "dotproduct_softmax":
        ones = F.unfold(torch.ones(1, 1, H, W, device=src.device, dtype=src.dtype), kernel_size=k, padding=d)
        inside = ones.view(1, k * k, H, W).permute(0, 2, 3, 1) > 0
        corr = corr.masked_fill(~inside, float("-inf")).softmax(dim=-1)
    return corr.view(N, H, W, k, k)


class STSSTransformation(nn.Module):
    def __init__(self, window=(5, 9, 9), corr_func: str = "cosine"):
        super().__init__()
        self.window, self.corr_func = tuple(window), corr_func

    def forward(self, x: Tensor, t: int, h: int, w: int) -> Tensor:
        """``x (B*t*h*w, C)`` -> ``(B, t, h, w, L, k, k)`` similarities.  The features stay token-major: the window
        kernel (``ops/stss.py``) reads neighbour vectors in place instead of unfolding ``L * k * k`` copies."""
        from ..ops.stss import local_window_correlation
        L, k, _ = self.window
        C = x.shape[-1]
        v = x.view(-1, t, h * w, C)
        B = v.shape[0]
        if self.corr_func == "cosine":
            v = F.normalize(v, p=2, dim=-1)
        elif self.corr_func not in ("dotproduct", "dotproduct_softmax"):
            raise ValueError(f"unknown corr_func {self.corr_func!r}")
        corr = local_window_correlation(v, t, h, w, L, k)                          # (B, t, hw, L, k*k)
        if self.corr_func != "cosine":
            corr = corr * C ** -0.5
        if self.corr_func == "dotproduct_softmax":
            ones = F.unfold(torch.ones(1, 1, h, w, device=x.device, dtype=corr.dtype), kernel_size=k, padding=k // 2)
            inside = ones.view(k * k, h * w).t() > 0                              # (hw, k*k)
            corr = corr.masked_fill(~inside[None, None, :, None, :], float("-inf")).softmax(dim=-1)
        return corr.view(B, t, h, w, max(L, 1), k, k)


class _Pointwise(nn.Sequential):
    """``Conv3d(1x1x1, bias=False) [+ norm] + GELU`` keeping the reference's sequential indices."""

    def __init__(self, c_in: int, c_out: int, norm: str | None, lead: int = 0):
        mods: list[nn.Module] = [nn.Identity() for _ in range(lead)]
        mods.append(nn.Conv3d(c_in, c_out, kernel_size=1, bias=False))
        if norm is not None:
            mods.append(_make_norm3d(c_out, norm))
        mods.append(nn.GELU())
        super().__init__(*mods)


class STSSExtraction(nn.Module):
    def __init__(self, window=(5, 9, 9), chnls=(256,), norm: str = "groupnorm"):
        super().__init__()
        self.window = tuple(window)
        self.conv0 = _Pointwise(window[1] * window[2], chnls[0], norm)

    def forward(self, s: Tensor) -> Tensor:
        """``(B, t, h, w, L, k, k)`` -> ``(B*L, C, t, h, w)``."""
        B, t, h, w, L, k, _ = s.shape
        x = s.permute(0, 4, 5, 6, 1, 2, 3).reshape(B * L, k * k, t, h, w)
        return self.conv0(x)


class STSSIntegration(nn.Module):
    def __init__(self, d_in: int, window=(5, 9, 9), chnls=(64, 64, 64), norm: str = "groupnorm", mode: str = "lite"):
        super().__init__()
        self.window, self.mode = tuple(window), mode
        L = window[0]
        if mode == "lite":
            self.fuse = _Pointwise(d_in * L, chnls[-1], None, lead=1)         # index 0 is the rearrange in the reference
            return
        def conv3(ci, co):
            return nn.Sequential(nn.Conv3d(ci, co, (1, 3, 3), padding=(0, 1, 1), bias=False), _make_norm3d(co, norm), nn.GELU())
        self.conv0, self.conv1 = conv3(d_in, chnls[0]), conv3(chnls[0], chnls[1])
        self.conv2_fuse = nn.Sequential(nn.Identity(), *conv3(chnls[1] * L, chnls[2]))

    def _merge(self, x: Tensor) -> Tensor:
        L = self.window[0]
        BL, C, t, h, w = x.shape
        return x.view(BL // L, L * C, t, h, w)

    def forward(self, x: Tensor) -> Tensor:
        if self.mode == "lite":
            return self.fuse(self._merge(x))
        x = self.conv1(self.conv0(x))
        return self.conv2_fuse(self._merge(x))


class STSSEncoder(nn.Module):
    def __init__(self, d_in: int, d_hid: int, d_out: int, window=(5, 9, 9), ext_chnls=(256,), int_chnls=(256, 256, 512),
                 corr_func: str = "cosine", norm: str = "groupnorm", int_mode: str = "lite"):
        super().__init__()
        self.ln_pre = nn.LayerNorm(d_in, eps=1e-6)
        self.in_proj = nn.Linear(d_in, d_hid)
        self.stss_transformation = STSSTransformation(window, corr_func)
        self.stss_extraction = STSSExtraction(window, ext_chnls, norm)
        self.stss_integration = STSSIntegration(ext_chnls[-1], window, int_chnls, norm, int_mode)
        self.out_proj = nn.Linear(int_chnls[-1], d_out)

    def forward(self, x: Tensor, t: int, h: int, w: int) -> Tensor:
        x = self.in_proj(self.ln_pre(x))
        s = self.stss_transformation(x, t, h, w)
        y = self.stss_integration(self.stss_extraction(s))                   # (B, C, t, h, w)
        return self.out_proj(y.permute(0, 2, 3, 4, 1).reshape(-1, y.shape[1]))


class MotionModule(nn.Module):
    def __init__(self, d_in: int, d_hid: int, d_out: int, window=(5, 9, 9), ext_chnls=(256,), int_chnls=(256, 256, 512),
                 corr_func: str = "cosine", n_encoders: int = 1, use_layerscale: bool = False, layerscale_init: float = 1e-5,
                 norm: str = "groupnorm", int_mode: str = "lite", zero_init_residual: bool = True):
        super().__init__()
        if len(window) != 3 or any(v < 1 or v % 2 == 0 for v in window):
            raise ValueError(f"window dims must be positive odd ints (L, kh, kw); got {window}.")
        if window[1] != window[2]:
            raise ValueError(f"window spatial dims must be square; got {window[1:]}.")
        self.use_layerscale, self.layerscale_init, self.zero_init_residual = use_layerscale, layerscale_init, zero_init_residual
        self.stss_encoders = nn.ModuleList([
            STSSEncoder(d_in if i == 0 else (d_out if use_layerscale else d_hid), d_hid, d_out if use_layerscale else d_hid,
                        window, ext_chnls, int_chnls, corr_func, norm, int_mode) for i in range(n_encoders)])
        if use_layerscale:
            self.layerscale = nn.Parameter(torch.ones(d_out) * layerscale_init)
        else:
            self.out_proj = nn.Linear(d_hid, d_out)
        self.initialize_weights()

    def initialize_weights(self) -> None:
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.trunc_normal_(m.weight, std=0.02)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
            elif isinstance(m, nn.Conv3d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
            elif isinstance(m, (nn.BatchNorm3d, nn.SyncBatchNorm, nn.LayerNorm, nn.GroupNorm)):
                nn.init.ones_(m.weight), nn.init.zeros_(m.bias)
        if self.use_layerscale:
            self.layerscale.data.fill_(0.0 if self.zero_init_residual else self.layerscale_init)
        elif self.zero_init_residual:
            nn.init.zeros_(self.out_proj.weight), nn.init.zeros_(self.out_proj.bias)

    def forward(self, x: Tensor, grid_sizes: Tensor) -> Tensor:
        """``x (sum_i T_i*H_i*W_i, C)`` in ``(b t h w)`` order, ``grid_sizes (B, 3)`` rows ``[T, H, W]`` -> residual."""
        def run(xv: Tensor, g) -> Tensor:
            t, h, w = (int(v) for v in g)
            out, acc = xv, None
            for enc in self.stss_encoders:
                out = enc(out, t, h, w)
                acc = out if acc is None else acc + out
            return acc
        if bool((grid_sizes == grid_sizes[0]).all()):
            out = run(x, grid_sizes[0])
        else:
            sizes = grid_sizes.prod(dim=1).tolist()
            out = torch.cat([run(xv, g) for xv, g in zip(x.split(sizes, 0), grid_sizes)], 0)
        return out * self.layerscale if self.use_layerscale else self.out_proj(out)


class RLDXVideoEncoder(nn.Module):
    """Per-frame SigLIP with the motion residual added after one encoder layer; returns the current frame's tokens.

    Padded history frames are replaced by the first real frame before the correlation (no spurious motion against a
    blank frame); ``T == 1`` is a plain single-frame pass.  The tower is shared with the policy, not owned.
    """

    def __init__(self, vision_tower: SiglipVisionModel, multi_modal_projector: nn.Module, max_num_frames: int,
                 gradient_checkpointing: bool = False, *, motion_insert_layer: int | None = None, motion_hidden_dim: int = 256,
                 motion_window=(5, 9, 9), motion_corr_func: str = "cosine", motion_n_encoders: int = 1,
                 motion_norm: str = "groupnorm", motion_int_mode: str = "lite", motion_zero_init: bool = True):
        super().__init__()
        if max_num_frames < 1:
            raise ValueError(f"max_num_frames ({max_num_frames}) must be >= 1.")
        self.max_num_frames, self.gradient_checkpointing = max_num_frames, gradient_checkpointing
        self._refs = [vision_tower, multi_modal_projector]                   # plain list: not registered as submodules
        cfg = vision_tower.vision_model.cfg
        n_patches = (cfg.image_size // cfg.patch_size) ** 2
        grid = int(round(n_patches ** 0.5))
        if grid * grid != n_patches:
            raise ValueError(f"Motion module requires a square patch grid; got {n_patches} patches.")
        if max(motion_window[1:]) > grid:
            raise ValueError(f"motion_window spatial size {tuple(motion_window[1:])} exceeds patch grid {grid}x{grid}.")
        n_layers = len(vision_tower.vision_model.encoder.layers)
        insert = n_layers // 3 if motion_insert_layer is None else motion_insert_layer
        if not 0 <= insert < n_layers:
            raise ValueError(f"motion_insert_layer ({insert}) out of range [0, {n_layers}).")
        self.num_video_tokens, self.motion_grid_hw, self.motion_insert_layer = n_patches, grid, insert
        self.motion_module = MotionModule(cfg.hidden_size, motion_hidden_dim, cfg.hidden_size, tuple(motion_window),
                                          corr_func=motion_corr_func, n_encoders=motion_n_encoders, norm=motion_norm,
                                          int_mode=motion_int_mode, zero_init_residual=motion_zero_init)

    @property
    def vision_tower(self) -> SiglipVisionModel:
        return self._refs[0]

    @property
    def multi_modal_projector(self) -> nn.Module:
        return self._refs[1]

    def _apply_motion(self, hidden: Tensor, b: int, t: int, is_pad: Tensor | None) -> Tensor:
        n, d = hidden.shape[1:]
        x = hidden.view(b, t, n, d)
        if is_pad is not None:
            real = ~is_pad.bool()
            real[:, -1] = True
            first = real.float().argmax(dim=1)
            fill = x[torch.arange(b, device=x.device), first]
            x = torch.where((~real)[:, :, None, None], fill[:, None], x)
        grid = torch.tensor([[t, self.motion_grid_hw, self.motion_grid_hw]] * b, dtype=torch.long, device=hidden.device)
        mm = self.motion_module
        dt = next(mm.parameters()).dtype
        res = mm(x.reshape(b * t * n, d).to(dt), grid)
        return hidden + res.view(b * t, n, d).to(hidden.dtype)

    def forward(self, video: Tensor, obs_history_is_pad: Tensor | None = None) -> Tensor:
        """``video (B, T, C, H, W)`` in [0, 1] -> ``(B, tokens, vlm_width)``."""
        if video.dim() != 5:
            raise ValueError(f"Expected 5D input (B, T, C, H, W); got {tuple(video.shape)}.")
        b, t = video.shape[:2]
        if not 1 <= t <= self.max_num_frames:
            raise ValueError(f"Expected 1 <= T <= max_num_frames ({self.max_num_frames}); got {t}.")
        vm = self.vision_tower.vision_model
        x = vm.embeddings((video * 2.0 - 1.0).flatten(0, 1), vm.post_layernorm.weight.dtype)
        ckpt = self.gradient_checkpointing and self.training and torch.is_grad_enabled()
        for i, layer in enumerate(vm.encoder.layers):
            if ckpt:
                from torch.utils.checkpoint import checkpoint
                x = checkpoint(layer, x, use_reentrant=False)
            else:
                x = layer(x)
            if t > 1 and i == self.motion_insert_layer:
                x = self._apply_motion(x, b, t, obs_history_is_pad)
        x = vm.post_layernorm(x)
        return self.multi_modal_projector(x.view(b, t, *x.shape[1:])[:, -1])
