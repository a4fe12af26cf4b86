"""pi0.5-MEM: pi0.5 with short-term visual memory (reference ``src/opentau/policies/pi05_mem/modeling_pi05.py:347-1695``).

Prefix: per camera the CURRENT frame's tokens of a video encoder that has seen ``T`` frames (bidirectional) | prompt |
``T`` state tokens, one per history step, padded steps masked (all bidirectional with the images) | FAST action
tokens (causal, training only).  Video patches get 2-D positions under interleaved MRoPE: a present video block uses
one temporal index and ``grid`` position units; text, state and action tokens have ``t == h == w``.  Suffix, losses
and sampler are those of pi0.5.
"""

from __future__ import annotations

from collections import deque
from typing import Any

import torch
from torch import Tensor

from ... import ops
from ...models.layers import Linear
from ...models.motion_module import RLDXVideoEncoder
from ...models.video_encoder import SpaceTimeSiglipVideoEncoder
from ..pi05.modeling_pi05 import PI05FlowMatching, PI05Policy
from .configuration_pi05_mem import PI05MemConfig


def build_mrope_prefix_positions(seg_masks: list[Tensor], seg_is_video: list[bool], grid: int) -> Tensor:
    """``(3, B, L)`` (temporal, height, width) positions of a prefix made of ordered segments.

    A video segment (``grid*grid`` row-major patches) shares one temporal index ``base`` and gets ``h = base + row``,
    ``w = base + col``; when present it advances the running position by ``grid``.  A text-style segment advances by
    one per real token with ``t == h == w``.
    """
    device = seg_masks[0].device
    B = seg_masks[0].shape[0]
    cur = torch.zeros(B, dtype=torch.long, device=device)
    idx = torch.arange(grid * grid, device=device)
    rows, cols = idx // grid, idx % grid
    blocks = []
    for mask, is_video in zip(seg_masks, seg_is_video, strict=True):
        n = mask.shape[1]
        if is_video:
            base = cur[:, None]
            blocks.append(torch.stack([base.expand(B, n), base + rows[None], base + cols[None]], 0))
            cur = cur + mask[:, 0].long() * grid
        else:
            pos = cur[:, None] + torch.cumsum(mask.long(), 1) - 1
            blocks.append(pos[None].expand(3, B, n))
            cur = cur + mask.long().sum(1)
    return torch.cat(blocks, dim=2)


class PI05MemFlowMatching(PI05FlowMatching):
    def __init__(self, config: PI05MemConfig, tokenizer=None):
        super().__init__(config, tokenizer)
        w = self.wrapper
        tower, proj = w.paligemma.vision_tower, w.paligemma.model.multi_modal_projector
        if config.use_motion:
            self.video_encoder = RLDXVideoEncoder(
                tower, proj, config.n_obs_steps, config.gradient_checkpointing,
                motion_insert_layer=config.motion_insert_layer, motion_hidden_dim=config.motion_hidden_dim,
                motion_window=tuple(config.motion_window), motion_corr_func=config.motion_corr_func,
                motion_n_encoders=config.motion_n_encoders, motion_norm=config.motion_norm,
                motion_int_mode=config.motion_int_mode, motion_zero_init=config.motion_zero_init)
        else:
            enc = SpaceTimeSiglipVideoEncoder(tower, max_num_frames=config.n_obs_steps,
                                              spacetime_layer_stride=config.spacetime_layer_stride)
            enc._modules.pop("vision")                      # the tower is owned by the backbone wrapper
            object.__setattr__(enc, "vision", tower)
            self.video_encoder = enc
        if not hasattr(self, "state_proj"):
            self.state_proj = Linear(config.max_state_dim, w.vlm_cfg.hidden_size, bias=True)
        vc = tower.vision_model.cfg
        self._video_grid = vc.image_size // vc.patch_size

    def discrete_block_len(self) -> int:
        return self.config.discrete_action_max_length

    def embed_video(self, video: Tensor, obs_history_is_pad: Tensor | None = None) -> Tensor:
        """``video (B, T, C, H, W)`` in [-1, 1] -> current-frame tokens ``(B, N, d)`` in backbone width."""
        if self.config.use_motion:
            return self.video_encoder((video + 1.0) * 0.5, obs_history_is_pad)
        valid = None if obs_history_is_pad is None else ~obs_history_is_pad.bool()
        feats = self.video_encoder(video, valid)
        return self.wrapper.paligemma.model.multi_modal_projector(feats)

    def embed_prefix(self, images, img_masks, lang_tokens, lang_masks, response_tokens=None, response_masks=None,
                     discrete_actions=None, discrete_action_masks=None, state=None, *, state_history=None,
                     obs_history_is_pad=None):
        w = self.wrapper
        dtype = w.da_head.weight.dtype
        device = lang_tokens.device
        B = lang_tokens.shape[0]
        embs, pads, att, is_video = [], [], [], []
        for vid, m in zip(images, img_masks):
            vid = vid if vid.dim() == 5 else vid[:, None]
            pad = obs_history_is_pad[:, -vid.shape[1]:] if obs_history_is_pad is not None else None
            e = self.embed_video(vid, pad).to(dtype)
            embs.append(e), pads.append(m[:, None].expand(B, e.shape[1])), is_video.append(True)
            att += [0] * e.shape[1]
        lang = w.embed_language_tokens(lang_tokens).to(dtype)
        embs.append(lang), pads.append(lang_masks.bool()), is_video.append(False)
        att += [0] * lang.shape[1]
        st = state_history if state_history is not None else state
        st = st if st.dim() == 3 else st[:, None]
        T = st.shape[1]
        if obs_history_is_pad is not None:
            s_mask = ~obs_history_is_pad.bool()[:, -T:]
        else:
            s_mask = torch.zeros(B, T, dtype=torch.bool, device=device)
        s_mask = s_mask.clone()
        s_mask[:, -1] = True                                # the current step is always real
        st = st.masked_fill(~s_mask[:, :, None], 0.0)
        embs.append(self.state_proj(st.to(self.state_proj.weight.dtype)).to(dtype))
        pads.append(s_mask), is_video.append(False)
        att += [0] * T
        if discrete_actions is not None:
            d = w.embed_discrete_actions(discrete_actions).to(dtype)
            embs.append(d), pads.append(discrete_action_masks.bool()), is_video.append(False)
            att += [1] * d.shape[1]
        pad_cat = torch.cat(pads, 1)
        att_t = self._const(("att", tuple(att), str(device)),
                            lambda: torch.tensor(att, dtype=torch.bool, device=device))[None].expand(B, -1)
        pos = build_mrope_prefix_positions(pads, is_video, self._video_grid) \
            if self.config.rope_type == "mrope_interleaved" else None
        return torch.cat(embs, 1), pad_cat, att_t, pos


class PI05MemPolicy(PI05Policy):
    config_class = PI05MemConfig
    name = "pi05_mem"
    model_class = PI05MemFlowMatching

    def reset(self) -> None:
        super().reset()
        n = (self.config.n_obs_steps - 1) * self.config.history_interval + 1
        self._history: deque = deque([], maxlen=n)

    # -- batch preparation ---------------------------------------------------------------------------
    def prepare_images(self, batch):
        """Keeps the history axis: each camera becomes ``(B, T, C, H, W)`` in [-1, 1]."""
        cfg = self.config
        keys = [k for k in cfg.image_features if not k.startswith("empty_camera")] or \
            sorted(k for k in batch if k.startswith("camera") and isinstance(batch[k], Tensor))
        images, masks = [], []
        pad_flags = batch.get("img_is_pad")
        for i, k in enumerate(k for k in keys if k in batch):
            img = batch[k]
            img = img if img.dim() == 5 else img[:, None]
            B, T = img.shape[:2]
            flat = img.flatten(0, 1)
            if tuple(flat.shape[-2:]) != tuple(cfg.resize_imgs_with_padding):
                flat = ops.resize_with_pad(flat.float(), cfg.resize_imgs_with_padding[1], cfg.resize_imgs_with_padding[0],
                                           pad_value=0.0)
            images.append((flat * 2.0 - 1.0).view(B, T, *flat.shape[1:]))
            masks.append(~pad_flags[:, i].bool() if pad_flags is not None
                         else torch.ones(B, dtype=torch.bool, device=img.device))
        if not images:
            raise ValueError("no camera images in the batch")
        for _ in range(cfg.empty_cameras):
            images.append(torch.full_like(images[-1], -1.0)), masks.append(torch.zeros_like(masks[-1]))
        return images, masks

    def prepare_language(self, batch):
        device = batch["state"].device
        if "lang_tokens" in batch:
            return batch["lang_tokens"].to(device), batch["lang_masks"].to(device).bool()
        tasks = batch["prompt"]
        tasks = [tasks] if isinstance(tasks, str) else list(tasks)
        # "<eos>" is spelled out: the tokenizer maps it to the separator id (reference pi05_mem/modeling_pi05.py:1051-1068)
        enc = self.language_tokenizer([f"Task: {t}<eos>Actions:" for t in tasks], padding="max_length",
                                      padding_side="right", max_length=self.config.prompt_max_length,
                                      return_tensors="pt", truncation=True)
        return enc["input_ids"].to(device), enc["attention_mask"].to(device).bool()

    def _prefix_kwargs(self, batch, nb) -> dict[str, Any]:
        st = nb["state"]
        return {"state_history": st if st.dim() == 3 else st[:, None],
                "obs_history_is_pad": batch.get("obs_history_is_pad")}

    # -- closed loop: the policy keeps the observation history itself ----------------------------------
    def _build_history_batch(self, batch: dict[str, Any]) -> dict[str, Any]:
        """Stacks the last ``n_obs_steps`` observations (every ``history_interval``-th step); steps before the
        start of the episode repeat the oldest observation and are flagged in ``obs_history_is_pad``."""
        cfg = self.config
        keys = [k for k, v in batch.items() if isinstance(v, Tensor) and (k.startswith("camera") or k == "state")]
        self._history.append({k: batch[k] for k in keys})
        hist = list(self._history)
        picks, pad = [], []
        for i in range(cfg.n_obs_steps):
            back = (cfg.n_obs_steps - 1 - i) * cfg.history_interval
            j = len(hist) - 1 - back
            picks.append(hist[max(j, 0)]), pad.append(j < 0)
        out = dict(batch)
        for k in keys:
            out[k] = torch.stack([p[k] for p in picks], dim=1)
        B = batch["state"].shape[0]
        out["obs_history_is_pad"] = torch.tensor(pad, dtype=torch.bool, device=batch["state"].device)[None].expand(B, -1)
        return out

    @torch.no_grad()
    def select_action(self, batch: dict[str, Any], noise: Tensor | None = None) -> Tensor:
        if batch["state"].dim() == 2:
            batch = self._build_history_batch(batch)
        return super().select_action(batch, noise)
