"""pi0.7 low-level controller: Gemma-3 + SpaceTime-SigLIP video history + flow-matching expert.

Prefix layout (reference ``src/opentau/policies/pi07/low_level/modeling_pi07_low_level.py:1611-2013``):

    videos (one bidirectional block per camera, current-frame tokens; with ``keep_history_tokens`` one block per
    camera AND frame, oldest first -- the long-context variant whose decoder sequence is split over GPUs by
    ``parallel/cp.py``) | prompt (causal) | "State: " |
    T per-step state tokens (bidirectional) | state end | response? | metadata? | ";\\n "? |
    "Subgoal: " + subgoal images (bidirectional per camera) + ", "? | FAST action tokens (training only)

Whether an optional block is present is decided for the whole batch AND for all ranks with one all-reduce
(:func:`..common.global_or_branch_decisions`), so every rank launches the same kernels and collectives.
Text after the images is causal; the expert/suffix path, losses and sampler are those of pi0.6.
"""

from __future__ import annotations

from typing import Any

import torch
from torch import Tensor

from .... import ops
from ....models.layers import Linear
from ....models.video_encoder import SpaceTimeSiglipVideoEncoder
from ...pi05.modeling_pi05 import PI05Policy
from ...pi06.modeling_pi06 import PI06FlowMatching
from ..common import global_or_branch_decisions
from .configuration_pi07_low_level import PI07LowLevelConfig


class PI07LowLevelFlowMatching(PI06FlowMatching):
    def __init__(self, config: PI07LowLevelConfig, tokenizer=None):
        super().__init__(config, tokenizer)
        w = self.wrapper
        self.video_encoder = SpaceTimeSiglipVideoEncoder(self._tower(), max_num_frames=max(
            1, config.n_obs_steps), spacetime_layer_stride=config.spacetime_layer_stride)
        # registering the encoder must not duplicate the tower's parameters in state_dict
        self.video_encoder._modules.pop("vision")
        object.__setattr__(self.video_encoder, "vision", self._tower())
        self.state_proj = Linear(config.max_state_dim, w.vlm_cfg.hidden_size, bias=True)
        self.sync_branches = True

    # -- pieces -------------------------------------------------------------------------------------
    def _tower(self):
        return self.wrapper.gemma3.model.vision_tower

    def _projector(self):
        return self.wrapper.gemma3.model.multi_modal_projector

    def embed_video(self, video: Tensor, frame_valid: Tensor | None) -> Tensor:
        """``video (B,T,C,H,W)`` -> projected current-frame tokens ``(B, tokens, d)``; with
        ``config.keep_history_tokens`` the tokens of all ``T`` frames, ``(B, T, tokens, d)``."""
        if getattr(self.config, "keep_history_tokens", False):
            feats = self.video_encoder(video, frame_valid, keep_history=True)       # (B, T, N, d)
            B, T = feats.shape[:2]
            out = self._projector()(feats.flatten(0, 1))
            return out.view(B, T, *out.shape[1:])
        feats = self.video_encoder(video, frame_valid)
        return self._projector()(feats)

    def _text(self, text: str, B: int, device) -> Tensor:
        return self._embed_indicator(text, B, device)

    def embed_prefix(self, images, img_masks, lang_tokens, lang_masks, response_tokens=None, response_masks=None,
                     discrete_actions=None, discrete_action_masks=None, state=None, *, state_history=None,
                     history_is_pad=None, metadata_tokens=None, metadata_masks=None, subgoal_images=None,
                     subgoal_masks=None):
        w = self.wrapper
        dtype = w.da_head.weight.dtype
        device = lang_tokens.device
        B = lang_tokens.shape[0]
        embs, pads, att = [], [], []

        def add(e: Tensor, m: Tensor, a: list[int]):
            embs.append(e.to(dtype)), pads.append(m), att.extend(a)

        ones = lambda n: torch.ones(B, n, dtype=torch.bool, device=device)  # noqa: E731
        frame_valid = None if history_is_pad is None else ~history_is_pad.bool()
        for img, m in zip(images, img_masks):
            vid = img if img.dim() == 5 else img[:, None]
            fv = frame_valid[:, -vid.shape[1]:] if frame_valid is not None else None
            e = self.embed_video(vid, fv)
            if e.dim() == 4:
                # long-context variant: every frame of every camera stays in the decoder as its own bidirectional
                # block, oldest first; a block sees the blocks before it (frame-block-causal), padded history
                # frames are masked out like padded cameras
                T, n = e.shape[1], e.shape[2]
                fm = m[:, None].expand(B, T) if fv is None else (m[:, None] & fv.bool())
                fm = fm.clone()
                fm[:, -1] = m                                   # the current frame is real whenever the camera is
                for t in range(T):
                    first = [1] if (embs or t > 0) else [0]
                    add(e[:, t], fm[:, t, None].expand(B, n), first + [0] * (n - 1))
                continue
            add(e, m[:, None].expand(B, e.shape[1]), [1] + [0] * (e.shape[1] - 1) if embs else [0] * e.shape[1])
        lang = w.embed_language_tokens(lang_tokens)
        add(lang, lang_masks.bool(), [1] * lang.shape[1])
        if state_history is not None:
            e = self._text("State: ", B, device)
            add(e, ones(e.shape[1]), [1] * e.shape[1])
            T = state_history.shape[1]
            st = self.state_proj(state_history.to(self.state_proj.weight.dtype))
            sm = ones(T) if frame_valid is None else frame_valid[:, -T:].clone()
            sm[:, -1] = True                                   # the current step is always real
            add(st, sm, [1] + [0] * (T - 1))
            e = self._text(":\n", B, device)
            add(e, ones(e.shape[1]), [1] * e.shape[1])
        # optional blocks: identical decisions on every rank
        fields = ("response", "metadata", "subgoal")
        present = (response_tokens is not None, metadata_tokens is not None, bool(subgoal_images))
        anys = (present[0] and bool(response_masks.any()), present[1] and bool(metadata_masks.any()),
                present[2] and bool(torch.stack(subgoal_masks).any()))
        has_resp, has_meta, has_sub = global_or_branch_decisions(present, anys, fields, device, self.sync_branches)
        if has_resp and response_tokens is not None:
            r = w.embed_language_tokens(response_tokens)
            add(r, response_masks.bool(), [1] * r.shape[1])
        if has_meta and metadata_tokens is not None:
            m = w.embed_language_tokens(metadata_tokens)
            add(m, metadata_masks.bool(), [1] * m.shape[1])
        if has_resp or has_meta:
            e = self._text(";\n ", B, device)
            add(e, ones(e.shape[1]), [1] * e.shape[1])
        if has_sub and subgoal_images:
            e = self._text("Subgoal: ", B, device)
            add(e, ones(e.shape[1]), [1] * e.shape[1])
            for img, m in zip(subgoal_images, subgoal_masks):
                g = w.embed_image(img)
                add(g, m[:, None].expand(B, g.shape[1]), [1] + [0] * (g.shape[1] - 1))
            e = self._text(", ", B, device)
            add(e, ones(e.shape[1]), [1] * e.shape[1])
        if discrete_actions is not None:
            d = w.embed_discrete_actions(discrete_actions)
            add(d, discrete_action_masks.bool(), [1] * d.shape[1])
        embs_t, pads_t = torch.cat(embs, 1), torch.cat(pads, 1)
        att_t = self._const(("att", tuple(att), str(device)),
                            lambda: torch.tensor(att, dtype=torch.bool, device=device))[None].expand(B, -1)
        return embs_t, pads_t, att_t, None


class PI07LowLevelPolicy(PI05Policy):
    config_class = PI07LowLevelConfig
    name = "pi07_low_level"
    model_class = PI07LowLevelFlowMatching
    _PER_GROUP_PROJECTION_PREFIXES = ("model.state_proj.", "model.action_in_proj.", "model.action_out_proj.")

    @staticmethod
    def _vocab_size(config) -> int:
        from ...pi06.modeling_pi06 import PI06Policy
        return PI06Policy._vocab_size(config)

    def prepare_images(self, batch):
        """Keeps the history axis: each camera is ``(B, T, C, H, W)`` scaled to [-1, 1]."""
        cfg = self.config
        keys = [k for k in cfg.image_features if not k.startswith("empty_camera")] or \
            sorted(k for k in batch if k.startswith("camera") and isinstance(batch[k], Tensor))
        images, masks = [], []
        pad_flags = batch.get("img_is_pad")
        for i, k in enumerate(k for k in keys if k in batch):
            img = batch[k]
            if img.dim() == 4:
                img = img[:, None]
            B, T = img.shape[:2]
            flat = img.flatten(0, 1)
            if tuple(flat.shape[-2:]) != tuple(cfg.resize_imgs_with_padding):
                flat = ops.resize_with_pad(flat.float(), cfg.resize_imgs_with_padding[1],
                                           cfg.resize_imgs_with_padding[0], pad_value=0.0)
            images.append((flat * 2.0 - 1.0).view(B, T, *flat.shape[1:]))
            masks.append(~pad_flags[:, i].bool() if pad_flags is not None
                         else torch.ones(B, dtype=torch.bool, device=img.device))
        if not images:
            raise ValueError("no camera images in the batch")
        return images, masks

    def prepare_language(self, batch):
        device = batch["state"].device
        if "lang_tokens" in batch:
            return batch["lang_tokens"].to(device), batch["lang_masks"].to(device).bool()
        tasks = batch["prompt"]
        tasks = [tasks] if isinstance(tasks, str) else list(tasks)
        enc = self.language_tokenizer([f"Task: {t}, " for t in tasks], padding="max_length", padding_side="right",
                                      max_length=self.config.prompt_max_length, return_tensors="pt", truncation=True)
        return enc["input_ids"].to(device), enc["attention_mask"].to(device).bool()

    def prepare_response(self, batch):
        """The subtask text conditions the controller (it is an input here, never a CE target)."""
        device = batch["state"].device
        if "response_tokens" in batch:
            return batch["response_tokens"].to(device), batch["response_masks"].to(device).bool()
        resp = batch.get("response")
        if resp is None:
            return None, None
        # "Subtask: {text}, " without special tokens; an empty subtask is an empty, fully masked segment
        # (reference pi07/low_level/modeling_pi07_low_level.py:1226-1258)
        enc = self.language_tokenizer([f"Subtask: {r}, " if r != "" else "" for r in resp], padding="max_length",
                                      padding_side="right", max_length=self.config.response_max_length,
                                      return_tensors="pt", truncation=True, add_special_tokens=False)
        mask = enc["attention_mask"].bool() & torch.tensor([bool(r) for r in resp])[:, None]
        return enc["input_ids"].to(device), mask.to(device)

    def prepare_metadata(self, batch) -> tuple[Tensor | None, Tensor | None]:
        """Episode metadata as one text segment per sample, tokenized to ``metadata_max_length``:
        ``"Metadata: Speed: 30,  Quality: 4,  Mistake: False,  Robot: so101,  FPS: 20,  Control: ee, "`` with only the
        fields that are present, in exactly this order and spelling (each field is ``"<Label>: <value>, "`` and the
        fields are joined by one more space: the string a checkpoint was trained on must be reproduced token for token;
        reference ``src/opentau/policies/pi07/low_level/modeling_pi07_low_level.py:1348-1430``).  ``speed`` / ``quality``
        / ``mistake`` / ``fps`` are tensors with a ``<key>_is_pad`` flag per sample (a padded entry is dropped; a tensor
        without its flag counts as present); ``robot_type`` / ``control_mode`` are strings, empty = absent.  A sample
        with no field gets an empty, fully masked segment; ``(None, None)`` when no sample has any."""
        device = batch["state"].device
        if "metadata_tokens" in batch:
            return batch["metadata_tokens"].to(device), batch["metadata_masks"].to(device).bool()
        B = batch["state"].shape[0]

        def numeric(key: str, i: int):
            if key not in batch:
                return None
            pad = batch.get(f"{key}_is_pad")
            if pad is not None and bool(pad[i]):
                return None
            v = batch[key][i]
            return v.item() if isinstance(v, Tensor) else v

        def text(key: str, i: int):
            v = batch.get(key)
            if v is None:
                return None
            v = v if isinstance(v, str) else v[i]
            return v or None

        rows: list[str] = []
        for i in range(B):
            segs = []
            for label, value in (("Speed", numeric("speed", i)), ("Quality", numeric("quality", i)),
                                 ("Mistake", numeric("mistake", i)), ("Robot", text("robot_type", i)),
                                 ("FPS", numeric("fps", i)), ("Control", text("control_mode", i))):
                if value is not None:
                    segs.append(f"{label}: {value}, ")
            rows.append(f"Metadata: {' '.join(segs)}" if segs else "")
        if not any(rows):
            return None, None
        enc = self.language_tokenizer(rows, padding="max_length", padding_side="right",
                                      max_length=self.config.metadata_max_length, return_tensors="pt",
                                      truncation=True, add_special_tokens=False)
        mask = enc["attention_mask"].bool() & torch.tensor([bool(r) for r in rows])[:, None]
        return enc["input_ids"].to(device), mask.to(device)

    def _prefix_kwargs(self, batch, nb) -> dict[str, Any]:
        device = nb["state"].device
        st = nb["state"]
        st = st if st.dim() == 3 else st[:, None]
        kw: dict[str, Any] = {"state_history": st, "history_is_pad": batch.get("obs_history_is_pad")}
        mt, mm = self.prepare_metadata(batch)
        kw["metadata_tokens"], kw["metadata_masks"] = mt, mm
        subs = sorted(k for k in batch if k.startswith("subgoal") and not k.endswith("_is_pad"))
        if subs:
            cfgsz = self.config.resize_imgs_with_padding
            imgs, ms = [], []
            for k in subs:
                im = batch[k].to(device)
                if tuple(im.shape[-2:]) != tuple(cfgsz):
                    im = ops.resize_with_pad(im.float(), cfgsz[1], cfgsz[0], pad_value=0.0)
                imgs.append(im * 2.0 - 1.0)
                pad = batch.get(f"{k}_is_pad")
                if pad is None:                       # datasets emit one flag for all cameras: subgoals are all-or-none
                    pad = batch.get("subgoal_is_pad")
                ms.append(~pad.bool().to(device) if pad is not None
                          else torch.ones(im.shape[0], dtype=torch.bool, device=device))
            kw["subgoal_images"], kw["subgoal_masks"] = imgs, ms
        return kw
