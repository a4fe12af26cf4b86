"""pi0.5: SigLIP + Gemma-2B backbone with a Gemma-300M flow-matching action expert.

Behaviour follows OpenTau ``src/opentau/policies/pi05/modeling_pi05.py`` (prefix layout ``:1370-1569``,
suffix ``:1571-1636``, training forward with knowledge insulation ``:1638-1878``, Euler sampler
``:1880-2120``), re-designed around static shapes:

* the prefix pass writes post-RoPE K/V into one pre-allocated cache tensor;
* the denoise loop runs a fixed ``num_steps`` times with no host round trip, so it can be replayed
  from a CUDA graph (``runtime.graphs``);
* all adaptive-norm modulations of the expert are produced by one GEMM per pass.

State-dict keys keep the reference names (``model.paligemma_with_expert.paligemma.model.language_model…``,
``…gemma_expert.model.layers.N…``, ``model.action_in_proj`` …).
"""

from __future__ import annotations

import math
from collections import deque
from typing import Any

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from ... import ops
from ...models.dual_stream import DualStreamDecoder, KVCache
from ...models.layers import Linear, Tower, TowerConfig
from ...datasets.action_indexing import add_chunk_start_state, subtract_chunk_start_state
from ...models.siglip import MultiModalProjector, SiglipConfig, SiglipVisionModel
from ...utils.tokenizer import load_action_tokenizer, load_text_tokenizer, pad_tokens
from ..normalize import Normalize, Unnormalize
from ..pretrained import PreTrainedPolicy
from .configuration_pi05 import PI05Config


def make_att_2d_masks(pad_masks: Tensor, att_masks: Tensor, n_cross_att_tokens: int | None = None,
                      cross_att_pad_masks: Tensor | None = None) -> Tensor:
    """Dense form of the block mask (kept for API parity and tests; kernels use block ids).

    Token i attends j iff both are valid and ``cumsum(att)[j] <= cumsum(att)[i]``; cross-attention
    columns are prepended and gated only by padding (``modeling_pi05.py:120-190``).
    """
    if att_masks.ndim != 2:
        raise ValueError(att_masks.ndim)
    if pad_masks.ndim != 2:
        raise ValueError(pad_masks.ndim)
    blk, valid = ops.make_block_ids(pad_masks, att_masks)
    m = ops.dense_mask_from_blocks(blk, blk, valid, valid)
    if n_cross_att_tokens is not None:
        assert cross_att_pad_masks is not None, "cross_att_pad_masks must be provided if n_cross_att_tokens is provided"
        assert cross_att_pad_masks.shape == (att_masks.size(0), n_cross_att_tokens)
        cross = valid[:, :, None] & cross_att_pad_masks.bool()[:, None, :]
        m = torch.cat([cross, m], dim=2)
    return m


def gemma_2b_config(**over) -> TowerConfig:
    return TowerConfig(**{**dict(hidden_size=2048, num_hidden_layers=18, num_attention_heads=8,
                                 num_key_value_heads=1, head_dim=256, intermediate_size=16384,
                                 vocab_size=257152, hidden_act="gelu_tanh"), **over})


def gemma_300m_config(**over) -> TowerConfig:
    return TowerConfig(**{**dict(hidden_size=1024, num_hidden_layers=18, num_attention_heads=8,
                                 num_key_value_heads=1, head_dim=256, intermediate_size=4096,
                                 vocab_size=257152, hidden_act="gelu_tanh", use_adarms=True,
                                 adarms_cond_dim=1024), **over})


class _PaliGemmaModel(nn.Module):
    def __init__(self, vlm: TowerConfig, vision: SiglipConfig):
        super().__init__()
        self.vision_tower = SiglipVisionModel(vision)
        self.multi_modal_projector = MultiModalProjector(vision.hidden_size, vlm.hidden_size)
        self.language_model = Tower(vlm, with_embed=True)


class _PaliGemma(nn.Module):
    """``paligemma.model.{vision_tower,multi_modal_projector,language_model}`` + tied ``lm_head``."""

    def __init__(self, vlm: TowerConfig, vision: SiglipConfig):
        super().__init__()
        self.model = _PaliGemmaModel(vlm, vision)

    @property
    def language_model(self) -> Tower:
        return self.model.language_model

    @property
    def vision_tower(self) -> SiglipVisionModel:
        return self.model.vision_tower

    def lm_head_weight(self) -> Tensor:
        return self.model.language_model.embed_tokens.weight


class _GemmaExpert(nn.Module):
    def __init__(self, cfg: TowerConfig):
        super().__init__()
        self.model = Tower(cfg, with_embed=False)


class PaliGemmaWithExpertModel(nn.Module):
    """Backbone + expert pair sharing attention (reference ``paligemma_with_expert.py:305-803``)."""

    def __init__(self, config: PI05Config):
        super().__init__()
        self.config = config
        vlm = gemma_2b_config(**(config.vlm or {}))
        exp_over = dict(config.expert or {})
        exp = gemma_300m_config(**exp_over)
        if "hidden_size" in exp_over and "adarms_cond_dim" not in exp_over:
            exp.adarms_cond_dim = exp.hidden_size
        vis = SiglipConfig(**{**dict(image_size=config.resize_imgs_with_padding[0]), **(config.vision or {})})
        self.vlm_cfg, self.expert_cfg, self.vision_cfg = vlm, exp, vis
        self.paligemma = _PaliGemma(vlm, vis)
        no_expert = bool(getattr(config, "disable_action_expert", False))      # text-only users (planners)
        self.gemma_expert = None if no_expert else _GemmaExpert(exp)
        self.discrete_action_embedding = nn.Embedding(config.discrete_action_vocab_size, vlm.hidden_size,
                                                      padding_idx=0)
        self.da_head = Linear(vlm.hidden_size, config.discrete_action_vocab_size, bias=True)
        towers = [self.paligemma.language_model] + ([] if no_expert else [self.gemma_expert.model])
        self.decoder = DualStreamDecoder(towers, dropout=config.dropout,
                                         gradient_checkpointing=config.gradient_checkpointing)
        self.set_requires_grad()

    # -- freezing ------------------------------------------------------------------------------
    def set_requires_grad(self) -> None:
        c = self.config
        if c.freeze_vision_encoder:
            self.paligemma.vision_tower.eval()
            for p in self.paligemma.vision_tower.parameters():
                p.requires_grad = False
        if c.train_expert_only:
            self.paligemma.eval()
            for p in self.paligemma.parameters():
                p.requires_grad = False
        if c.train_vision_encoder_only:
            for p in self.parameters():
                p.requires_grad = False
            for p in self.paligemma.vision_tower.parameters():
                p.requires_grad = True
            for p in self.paligemma.model.multi_modal_projector.parameters():
                p.requires_grad = True
        if c.train_state_action_representation_only:
            for p in self.parameters():
                p.requires_grad = False
            for p in list(self.discrete_action_embedding.parameters()) + list(self.da_head.parameters()):
                p.requires_grad = True

    def train(self, mode: bool = True):
        super().train(mode)
        if self.config.freeze_vision_encoder:
            self.paligemma.vision_tower.eval()
        if self.config.train_expert_only:
            self.paligemma.eval()
        if getattr(self.config, "train_state_action_representation_only", False):
            from ..utils import set_with_expert_train_mode_for_state_action_representation_only
            set_with_expert_train_mode_for_state_action_representation_only(self, mode)
        return self

    # -- embedders -----------------------------------------------------------------------------
    def embed_image(self, image: Tensor) -> Tensor:
        feats = self.paligemma.vision_tower(image)
        return self.paligemma.model.multi_modal_projector(feats)

    def embed_language_tokens(self, tokens: Tensor) -> Tensor:
        """Token embeddings already multiplied by ``sqrt(hidden)`` (the PaliGemma convention)."""
        return self.paligemma.language_model.embed(tokens)

    def lm_head_weight(self) -> Tensor:
        return self.paligemma.lm_head_weight()

    def embed_discrete_actions(self, actions: Tensor) -> Tensor:
        return ops.embedding(self.discrete_action_embedding.weight, actions, padding_idx=0)

    def forward(self, inputs_embeds, position_ids, q_blk, q_valid, **kw):
        if len(self.decoder.towers) == 1:                   # expert disabled: callers still pass / unpack a pair
            outs, cache = self.decoder([inputs_embeds[0]], position_ids, q_blk, q_valid, **{
                k: ([v[0]] if k == "adarms_cond" and v is not None else v) for k, v in kw.items()})
            return [outs[0], None], cache
        return self.decoder(inputs_embeds, position_ids, q_blk, q_valid, **kw)


class PI05FlowMatching(nn.Module):
    def __init__(self, config: PI05Config, tokenizer=None):
        super().__init__()
        self.config = config
        self.language_tokenizer = tokenizer
        setattr(self, self.wrapper_attr, self.build_wrapper(config))
        vlm_d = self.wrapper.vlm_cfg.hidden_size
        w = self.wrapper.expert_cfg.hidden_size
        if config.state_type == "continuous":
            self.state_proj = Linear(config.max_state_dim, vlm_d, bias=True)
        self.action_in_proj = Linear(config.max_action_dim, w, bias=True)
        self.action_out_proj = Linear(w, config.max_action_dim, bias=True)
        self.time_mlp_in = Linear(w, w, bias=True)
        self.time_mlp_out = Linear(w, w, bias=True)
        if config.use_modality_embedding:
            self.modality_embedding = nn.Embedding(5, vlm_d)
            self.action_modality_embedding = nn.Embedding(1, w)
            nn.init.zeros_(self.modality_embedding.weight)
            nn.init.zeros_(self.action_modality_embedding.weight)
        self._indicator_cache: dict[str, list[int]] = {}

    wrapper_attr = "paligemma_with_expert"

    def build_wrapper(self, config):
        return PaliGemmaWithExpertModel(config)

    @property
    def wrapper(self):
        """The backbone+expert pair (its attribute name is part of the checkpoint key contract)."""
        return getattr(self, self.wrapper_attr)

    def discrete_block_len(self) -> int:
        """Number of trailing prefix tokens that hold the discrete-action block (excluded from the KV
        cache the expert reads, so training and inference prefixes match)."""
        return self.config.discrete_action_indicator_max_length + self.config.discrete_action_max_length

    # -- sampling helpers ------------------------------------------------------------------------
    @staticmethod
    def sample_noise(shape, device) -> Tensor:
        return torch.randn(shape, dtype=torch.float32, device=device)

    @staticmethod
    def sample_time(bsize: int, device) -> Tensor:
        """``Beta(1.5, 1) * 0.999 + 0.001``; Beta(a,1) is ``U^(1/a)``, sampled on the device."""
        u = torch.rand(bsize, dtype=torch.float32, device=device).clamp_min(1e-12)
        return u.pow(1.0 / 1.5) * 0.999 + 0.001

    def _const(self, key, build) -> Tensor:
        """Device-resident constants (layout masks, indicator ids) are built once, so that repeated calls do
        no host-to-device copies and the whole sampler can be replayed from a CUDA graph."""
        cache = self.__dict__.setdefault("_const_cache", {})
        if key not in cache:
            cache[key] = build()
        return cache[key]

    def _indicator(self, text: str) -> list[int]:
        if text not in self._indicator_cache:
            self._indicator_cache[text] = list(self.language_tokenizer.encode(text, add_special_tokens=False))
        return self._indicator_cache[text]

    def _embed_indicator(self, text: str, bsize: int, device, max_len: int | None = None) -> Tensor:
        ids = self._indicator(text)
        if max_len is not None:
            ids = (ids + [0] * max_len)[:max_len] if len(ids) != max_len else ids
        tok = self._const(("ind", text, max_len, str(device)),
                          lambda: torch.tensor([ids], device=device)).expand(bsize, -1)
        return self.wrapper.embed_language_tokens(tok)

    # -- prefix / suffix -----------------------------------------------------------------------------
    def embed_prefix(self, images: list[Tensor], img_masks: list[Tensor], lang_tokens: Tensor, lang_masks: Tensor,
                     response_tokens: Tensor | None = None, response_masks: Tensor | None = None,
                     discrete_actions: Tensor | None = None, discrete_action_masks: Tensor | None = None,
                     state: Tensor | None = None):
        """Returns ``(embs, pad_masks, att_masks, segment_ids)``; att 0 joins the previous block."""
        pwe = self.wrapper
        dtype = pwe.paligemma.language_model.embed_tokens.weight.dtype
        device = lang_tokens.device
        B = lang_tokens.shape[0]
        embs, pads, att, seg = [], [], [], []
        if images:
            # all cameras in one vision pass: (B*cams, C, H, W)
            stacked = torch.stack(images, dim=1).flatten(0, 1)
            img_emb = pwe.embed_image(stacked).to(dtype)
            n_img = img_emb.shape[1]
            embs.append(img_emb.view(B, len(images) * n_img, -1))
            pads.append(torch.stack(img_masks, dim=1)[:, :, None].expand(B, len(images), n_img).reshape(B, -1))
            att += [0] * (len(images) * n_img)
            seg += [0] * (len(images) * n_img)
        lang = pwe.embed_language_tokens(lang_tokens)
        embs.append(lang)
        pads.append(lang_masks.bool())
        att += [0] * lang.shape[1]
        seg += [1] * lang.shape[1]
        ones = lambda n: torch.ones(B, n, dtype=torch.bool, device=device)  # noqa: E731
        if self.config.state_type == "continuous" and state is not None:
            e = self._embed_indicator("State: ", B, device)
            embs.append(e), pads.append(ones(e.shape[1]))
            att += [0] * e.shape[1]
            seg += [2] * e.shape[1]
            embs.append(self.state_proj(state.to(dtype))[:, None, :]), pads.append(ones(1))
            att += [0]
            seg += [2]
            e = self._embed_indicator(":\n", B, device)
            embs.append(e), pads.append(ones(e.shape[1]))
            att += [0] * e.shape[1]
            seg += [2] * e.shape[1]
        if self.config.predict_response:
            e = self._embed_indicator("Response: ", B, device, self.config.response_indicator_max_length)
            embs.append(e), pads.append(ones(e.shape[1]))
            att += [1] * e.shape[1]
            seg += [3] * e.shape[1]
        if response_tokens is not None:
            r = pwe.embed_language_tokens(response_tokens)
            embs.append(r), pads.append(response_masks.bool())
            att += [1] * r.shape[1]
            seg += [3] * r.shape[1]
        if discrete_actions is not None:
            e = self._embed_indicator("Action: ", B, device, self.config.discrete_action_indicator_max_length)
            embs.append(e), pads.append(ones(e.shape[1]))
            att += [1] * e.shape[1]
            seg += [4] * e.shape[1]
            d = pwe.embed_discrete_actions(discrete_actions).to(dtype)
            embs.append(d), pads.append(discrete_action_masks.bool())
            att += [1] * d.shape[1]
            seg += [4] * d.shape[1]
        embs_t = torch.cat(embs, dim=1)
        pads_t = torch.cat(pads, dim=1)
        att_t = self._const(("att", tuple(att), str(device)),
                            lambda: torch.tensor(att, dtype=torch.bool, device=device))[None].expand(B, -1)
        seg_t = self._const(("seg", tuple(seg), str(device)),
                            lambda: torch.tensor(seg, dtype=torch.long, device=device))[None].expand(B, -1)
        if self.config.use_modality_embedding:
            embs_t = embs_t + self.modality_embedding(seg_t).to(embs_t.dtype)
        return embs_t, pads_t, att_t, seg_t

    def embed_suffix(self, noisy_actions: Tensor, timestep: Tensor):
        """Returns ``(embs, pad_masks, att_masks, adarms_cond)``; time enters only through AdaRMS."""
        dtype = self.action_in_proj.weight.dtype
        B = noisy_actions.shape[0]
        device = noisy_actions.device
        w = self.action_in_proj.out_features
        time_emb = ops.sinusoidal_time_embedding(timestep, w, 4e-3, 4.0, out_dtype=dtype)
        action_emb = self.action_in_proj(noisy_actions.to(dtype))
        x = F.silu(self.time_mlp_in(time_emb))
        cond = F.silu(self.time_mlp_out(x))
        if self.config.use_modality_embedding:
            action_emb = action_emb + self.action_modality_embedding.weight.to(action_emb.dtype)
        T = action_emb.shape[1]
        pad = torch.ones(B, T, dtype=torch.bool, device=device)
        att = torch.zeros(B, T, dtype=torch.bool, device=device)
        att[:, 0] = True
        return action_emb, pad, att, cond

    # -- training ----------------------------------------------------------------------------------
    def forward(self, images, img_masks, lang_tokens, lang_masks, actions, actions_is_pad=None,
                response_tokens=None, response_masks=None, noise=None, time=None, discrete_actions=None,
                discrete_action_masks=None, state=None, real_action_dim=None, return_per_sample=False,
                prefix_kwargs=None):
        cfg = self.config
        pwe = self.wrapper
        prefix_embs, prefix_pad, prefix_att, pos = self.embed_prefix(
            images, img_masks, lang_tokens, lang_masks, response_tokens, response_masks, discrete_actions,
            discrete_action_masks, state=state, **(prefix_kwargs or {}))
        blk, valid = ops.make_block_ids(prefix_pad, prefix_att)
        if pos is None:
            pos = torch.cumsum(prefix_pad, dim=1) - 1
        mrope = pos.dim() == 3          # (3, B, L): interleaved multimodal RoPE, else one scalar position per token
        n_disc = self.discrete_block_len() if discrete_actions is not None else 0
        n_cross = prefix_embs.shape[1] - n_disc
        cp = getattr(self, "context_parallel", None)
        if cp is not None and cp.world > 1:
            prefix_out, cache = self._prefix_pass_context_parallel(cp, prefix_embs, pos, blk, valid, n_cross, mrope)
        else:
            (prefix_out, _), cache = pwe(inputs_embeds=[prefix_embs, None], position_ids=pos, q_blk=blk,
                                         q_valid=valid, fill_cache_len=n_cross, mrope=mrope)

        B = actions.shape[0]
        device = actions.device
        actions = actions.float()
        if noise is None:
            noise = self.sample_noise(actions.shape, device)
        if time is None:
            time = self.sample_time(B, device)
        if cfg.max_delay > 0:
            delay = torch.randint(0, cfg.max_delay + 1, (B,), device=device)
            frozen = torch.arange(cfg.chunk_size, device=device)[None, :] < delay[:, None]
        else:
            frozen = torch.zeros(B, cfg.chunk_size, dtype=torch.bool, device=device)
        time2 = torch.where(frozen, torch.zeros((), device=device), time[:, None])
        x_t, u_t = ops.flow_interpolate(actions, noise.float(), time2)

        suffix_embs, suffix_pad, suffix_att, cond = self.embed_suffix(x_t, time2)
        s_blk, s_valid = ops.make_block_ids(suffix_pad, suffix_att)
        offsets = self.suffix_offset(pos, prefix_pad, n_cross)
        s_pos = offsets + torch.cumsum(suffix_pad, dim=1) - 1
        if mrope:
            s_pos = s_pos[None].expand(3, -1, -1)
        if cfg.knowledge_insulation:
            cache = cache.detach()
        (_, suffix_out), _ = pwe(inputs_embeds=[None, suffix_embs], position_ids=s_pos, q_blk=s_blk,
                                 q_valid=s_valid, past=cache, adarms_cond=[None, cond], mrope=mrope)
        v_t = self.action_out_proj(suffix_out[:, -cfg.chunk_size:]).float()
        mse = ops.flow_matching_masked_mse(u_t, v_t, frozen, actions_is_pad, real_action_dim, return_per_sample)
        mse_loss, mse_ps = mse if return_per_sample else (mse, None)

        ce_ps = None
        if discrete_actions is not None:
            L = discrete_actions.shape[1]
            h = prefix_out[:, -(L + 1):-1]
            tok_ce = ops.linear_cross_entropy(h.reshape(B * L, -1), pwe.da_head.weight, pwe.da_head.bias,
                                              discrete_actions.reshape(-1)).view(B, L)
            tok_ce = tok_ce * discrete_action_masks.to(tok_ce.dtype)
            if return_per_sample:
                ce_ps = (tok_ce.sum(1), discrete_action_masks.sum(1).float())
            ce_loss = tok_ce.mean()
        else:
            ce_loss = torch.zeros((), device=device)
        if cfg.predict_response and response_tokens is not None:
            Lr = response_tokens.shape[1]
            start = -cfg.response_max_length - n_disc
            end = -n_disc - 1 if n_disc else -1
            h = prefix_out[:, start:end]
            labels = response_tokens[:, 1:]
            r_ce = ops.linear_cross_entropy(h.reshape(B * (Lr - 1), -1), pwe.lm_head_weight(), None,
                                            labels.reshape(-1)).view(B, Lr - 1)
            r_mask = response_masks[:, 1:].to(r_ce.dtype)
            r_ce = r_ce * r_mask
            if return_per_sample:
                add = (r_ce.sum(1), r_mask.sum(1))
                ce_ps = add if ce_ps is None else (ce_ps[0] + add[0], ce_ps[1] + add[1])
            ce_loss = ce_loss + r_ce.mean()
        out = {"MSE": mse_loss, "CE": ce_loss}
        if return_per_sample:
            out["MSE_per_sample"], out["CE_per_sample"] = mse_ps, ce_ps
        return out

    def _prefix_pass_context_parallel(self, cp, prefix_embs, pos, blk, valid, n_cross: int, mrope: bool):
        """The backbone's prefix pass with every sequence split over the ranks of ``cp``.

        Embeddings, masks and losses stay per sample (each rank has its own samples); only the decoder layers see
        the other layout, "all samples of the group, my slice of every sequence": the embeddings go through one
        all-to-all before layer 0 and the hidden states through the opposite one after the last layer (both
        differentiable), block-causal attention runs across the ranks inside the layers
        (``parallel/cp.py``), and the per-layer keys / values come back per sample for the action expert, which
        then runs on this rank's samples alone.  The reference has no counterpart (it drops history tokens before
        the decoder, ``policies/pi07/video_encoder.py:767-778``).  Needs knowledge insulation: the cache exchange
        carries no gradient."""
        if not self.config.knowledge_insulation:
            raise NotImplementedError("context parallelism needs knowledge_insulation (the prefix cache is detached)")
        W, r = cp.world, cp.rank
        B, S, _ = prefix_embs.shape
        pad = (-S) % (W * 8)                                 # slices of equal length, 16-byte rows for the kernels
        if pad:
            prefix_embs = torch.nn.functional.pad(prefix_embs, (0, 0, 0, pad))
            blk = torch.nn.functional.pad(blk, (0, pad), value=int(blk.max()) + 1)
            valid = torch.nn.functional.pad(valid, (0, pad), value=False)
            pos = torch.nn.functional.pad(pos, (0, pad))
        Sp = S + pad
        Sl = Sp // W
        x = cp.seq_scatter(prefix_embs)                                      # (W*B, Sl, d)
        blk_all = cp.batch_all_gather(blk.contiguous())                      # (W*B, Sp)
        valid_all = cp.batch_all_gather(valid.to(torch.uint8).contiguous()).bool()
        pos_all = cp.batch_all_gather(pos.contiguous(), dim=1 if mrope else 0)
        sl = slice(r * Sl, (r + 1) * Sl)
        (out_l, _), cache_l = self.wrapper(
            inputs_embeds=[x, None], position_ids=pos_all[..., sl].contiguous(), q_blk=blk_all[:, sl].contiguous(),
            q_valid=valid_all[:, sl].contiguous(), k_blk=blk_all, k_valid=valid_all, fill_cache_len=Sl, mrope=mrope,
            cp=cp)
        prefix_out = cp.seq_gather(out_l)[:, :S]
        with torch.no_grad():
            # (L, W*B, Sl, Hkv, D) -> per layer (B, Sp, Hkv, D) for this rank's samples; one exchange for all layers
            L = cache_l.k.shape[0]
            kv = torch.stack([cache_l.k.detach(), cache_l.v.detach()])       # (2, L, W*B, Sl, Hkv, D)
            kv = kv.permute(2, 3, 0, 1, 4, 5).contiguous()                   # (W*B, Sl, 2, L, Hkv, D)
            kv = cp._exchange(kv, scatter=False)                             # (B, Sp, 2, L, Hkv, D)
            kv = kv[:, :n_cross].permute(2, 3, 0, 1, 4, 5).contiguous()      # (2, L, B, n_cross, Hkv, D)
            cache = KVCache(kv[0], kv[1], valid[:, :n_cross].contiguous(), n_cross)
        return prefix_out, cache

    # -- inference ---------------------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, images, img_masks, lang_tokens, lang_masks, state=None,
                prefix_kwargs=None) -> tuple[KVCache, Tensor]:
        """Prefix pass: returns the KV cache and the per-sample count of valid prefix tokens."""
        prefix_embs, prefix_pad, prefix_att, pos = self.embed_prefix(images, img_masks, lang_tokens, lang_masks,
                                                                     state=state, **(prefix_kwargs or {}))
        blk, valid = ops.make_block_ids(prefix_pad, prefix_att)
        if pos is None:
            pos = torch.cumsum(prefix_pad, dim=1) - 1
        self._mrope = pos.dim() == 3
        _, cache = self.wrapper(inputs_embeds=[prefix_embs, None], position_ids=pos, q_blk=blk,
                                              q_valid=valid, fill_cache_len=prefix_embs.shape[1], mrope=self._mrope,
                                              cache_room=self.config.chunk_size + 8 + self._response_room())
        return cache, self.suffix_offset(pos, prefix_pad, prefix_embs.shape[1])   # (the suffix appends in place)

    def _response_room(self) -> int:
        return int(self.config.response_max_length) if self.config.predict_response else 0

    @torch.no_grad()
    def generate_response(self, cache: KVCache, prefix_len: Tensor) -> tuple[KVCache, Tensor, Tensor, Tensor]:
        """Greedy decoding of the response (the subtask / reasoning text) behind the cached prefix, one token per pass
        of the backbone alone, each token's keys / values appended to the cache so that the action expert then attends
        to the generated text (reference ``src/opentau/policies/pi05/modeling_pi05.py:1974-1999, 2122-2236``).

        The first token is ``<bos>``; every later one is the arg-max of the language head on the previous token's
        output.  Once a sample has produced ``<eos>`` (or a pad) its further tokens are pads, marked invalid in the
        cache and given no position.  Always ``response_max_length`` passes, no host synchronisation, so the loop can
        be captured in a CUDA graph.  Returns the longer cache, the per-sample first position of the action suffix,
        the tokens ``(B, L)`` and their validity mask."""
        cfg, pwe, tok = self.config, self.wrapper, self.language_tokenizer
        B, device = prefix_len.shape[0], prefix_len.device
        bos, eos, pad = tok.bos_token_id, tok.eos_token_id, tok.pad_token_id
        if bos is None or eos is None or pad is None:
            raise ValueError("response generation needs a tokenizer with bos, eos and pad ids")
        mrope = getattr(self, "_mrope", False)
        tokens = torch.empty(B, 0, dtype=torch.long, device=device)
        masks = torch.empty(B, 0, dtype=torch.bool, device=device)
        offset = prefix_len.clone()
        out = None
        for step in range(cfg.response_max_length):
            if step == 0:
                nxt = torch.full((B, 1), bos, dtype=torch.long, device=device)
            else:
                nxt = ops.linear(out[:, -1:], pwe.lm_head_weight()).float().argmax(dim=-1)
            if tokens.shape[1] > 1:
                done = ((tokens == eos) | (tokens == pad)).any(dim=1, keepdim=True)
                live = ~done
                nxt = torch.where(live, nxt, torch.full_like(nxt, pad))
            else:
                live = torch.ones(B, 1, dtype=torch.bool, device=device)
            tokens, masks = torch.cat([tokens, nxt], 1), torch.cat([masks, live], 1)
            emb = pwe.embed_language_tokens(nxt)
            pos = offset                                            # a finished sample's pad takes no new position
            offset = offset + live.long()
            blk, valid = ops.make_block_ids(live, torch.ones(B, 1, dtype=torch.long, device=device))
            (out, _), new = self.wrapper(inputs_embeds=[emb, None], position_ids=pos[None].expand(3, -1, -1) if mrope else pos,
                                         q_blk=blk, q_valid=valid, past=cache, fill_cache_len=1, mrope=mrope)
            cache = self._append_cache(cache, new, live)
        return cache, offset, tokens, masks

    @staticmethod
    def _append_cache(cache: KVCache, new: KVCache, valid: Tensor) -> KVCache:
        """``cache`` with the ``new.length`` tokens of ``new`` behind it: in place while the buffers have room."""
        n, at = new.length, cache.length
        if cache.writable_room() >= n:
            k, v = cache.k, cache.v
            k[:, :, at:at + n].copy_(new.k[:, :, :n])
            v[:, :, at:at + n].copy_(new.v[:, :, :n])
        else:
            k = torch.cat([cache.k[:, :, :at], new.k[:, :, :n]], dim=2)
            v = torch.cat([cache.v[:, :, :at], new.v[:, :, :n]], dim=2)
        return KVCache(k, v, torch.cat([cache.valid[:, :at], valid], dim=1), at + n)

    @staticmethod
    def suffix_offset(pos: Tensor, prefix_pad: Tensor, n_cross: int) -> Tensor:
        """First position of the suffix, ``(B, 1)``: the count of real cached tokens for scalar positions; for
        3-axis positions the largest position any real cached token uses, plus one (a video block compacts its
        ``grid x grid`` patches into ``grid`` position units, so the token count would leave a gap)."""
        if pos.dim() == 2:
            return prefix_pad[:, :n_cross].sum(-1, keepdim=True)
        cross = pos[:, :, :n_cross]
        real = torch.where(prefix_pad[None, :, :n_cross], cross, torch.full_like(cross, -1))
        return real.amax(dim=(0, 2))[:, None] + 1

    @torch.no_grad()
    def denoise_step(self, cache: KVCache, prefix_len: Tensor, x_t: Tensor, time: Tensor) -> Tensor:
        """One expert pass against the cached prefix: returns the velocity ``v_t`` (fp32)."""
        suffix_embs, suffix_pad, suffix_att, cond = self.embed_suffix(x_t, time)
        s_blk, s_valid = ops.make_block_ids(suffix_pad, suffix_att)
        s_pos = prefix_len + torch.cumsum(suffix_pad, dim=1) - 1
        mrope = getattr(self, "_mrope", False)
        if mrope:
            s_pos = s_pos[None].expand(3, -1, -1)
        (_, suffix_out), _ = self.wrapper(
            inputs_embeds=[None, suffix_embs], position_ids=s_pos, q_blk=s_blk, q_valid=s_valid, past=cache,
            adarms_cond=[None, cond], mrope=mrope)
        return self.action_out_proj(suffix_out[:, -self.config.chunk_size:]).float()

    def frozen_mask(self, delay: Tensor | int, batch: int, device) -> Tensor:
        """``(B, chunk)`` bool: chunk rows fixed by real-time chunking (the first ``delay`` rows)."""
        c = self.config.chunk_size
        if isinstance(delay, int):
            m = torch.zeros(1, c, dtype=torch.bool, device=device)
            if delay > 0:
                m[:, :delay] = True
            return m.expand(batch, -1)
        d = delay.to(device).reshape(-1, 1)
        return (torch.arange(c, device=device)[None, :] < d).expand(batch, -1)

    def executed_rows(self, delay: Tensor | int, batch: int, device, frozen: Tensor | None = None) -> Tensor:
        """``(B, chunk)`` bool: rows that reach the robot (not frozen, inside ``[delay, delay + n_action_steps)``);
        shared by the accel meter and the candidate critic so that the two score the same rows."""
        from ..accel import executed_row_mask
        if frozen is None:
            frozen = self.frozen_mask(delay, batch, device)
        if isinstance(delay, Tensor) and delay.ndim and 1 < delay.numel() < batch:
            delay = delay.repeat_interleave(batch // delay.numel())     # candidates: rows i*n .. i*n+n-1 share a delay
        return executed_row_mask(prefix_mask=frozen, delay=delay, chunk_size=self.config.chunk_size,
                                 n_action_steps=self.config.n_action_steps, device=device)

    @torch.no_grad()
    def denoise_loop(self, cache: KVCache, prefix_len: Tensor, noise: Tensor, action_prefix: Tensor | None = None,
                     delay: Tensor | int = 0, accel=None, frozen: Tensor | None = None) -> Tensor:
        """``num_steps`` Euler steps from t=1 to t=0 with a fixed trip count and device-only operations
        (no host round trip, no host-to-device copy), so the loop can be captured in a CUDA graph."""
        cfg = self.config
        n = cfg.num_steps
        dt = -1.0 / n
        x_t = noise.float().clone()
        B = x_t.shape[0]
        device = x_t.device
        if frozen is None:
            frozen = self.frozen_mask(delay, B, device)
        live = (~frozen).to(torch.float32)
        if accel is not None:
            accel.set_row_mask(self.executed_rows(delay, B, device, frozen))
        has_prefix = action_prefix is not None
        if has_prefix:               # committed actions enter every step unchanged ...
            x_t = torch.where(frozen[:, :, None], action_prefix.to(x_t.dtype), x_t)
        for i in range(n):
            t = 1.0 + i * dt
            time = live * t          # frozen rows run at diffusion time 0
            v_t = self.denoise_step(cache, prefix_len, x_t, time)
            if accel is not None:
                accel.update(v_t)
            # ... and are restored by the same kernel that takes the Euler step
            x_t = ops.euler_step(x_t, v_t, dt, frozen if has_prefix else None, action_prefix)
        return x_t

    @torch.no_grad()
    def sample_actions(self, images, img_masks, lang_tokens, lang_masks, action_prefix=None, delay=0,
                       noise=None, state=None, n_candidates: int = 1, accel=None, frozen=None,
                       prefix_kwargs=None) -> Tensor:
        B = lang_tokens.shape[0]
        device = lang_tokens.device
        cfg = self.config
        if noise is None:
            noise = self.sample_noise((B * n_candidates, cfg.chunk_size, cfg.max_action_dim), device)
        elif noise.shape[0] != B * n_candidates:
            raise ValueError(f"n_candidates={n_candidates} needs noise with {B * n_candidates} rows "
                             f"(got {tuple(noise.shape)})")
        cache, prefix_len = self.prefill(images, img_masks, lang_tokens, lang_masks, state=state,
                                         prefix_kwargs=prefix_kwargs)
        self.last_response_tokens = self.last_response_masks = None
        if cfg.predict_response:
            # before the candidates fan out: the decode is greedy and independent of the noise, so all candidates
            # share one response, and it extends the very cache that is widened below
            cache, prefix_len, self.last_response_tokens, self.last_response_masks = self.generate_response(cache, prefix_len)
        if n_candidates > 1:
            cache = cache.expand_batch(n_candidates)
            prefix_len = prefix_len.repeat_interleave(n_candidates, 0)
            if action_prefix is not None:
                action_prefix = action_prefix.repeat_interleave(n_candidates, 0)
            if frozen is not None:
                frozen = frozen.repeat_interleave(n_candidates, 0)
        return self.denoise_loop(cache, prefix_len, noise, action_prefix, delay, accel, frozen)


class PI05Policy(PreTrainedPolicy):
    """Policy wrapper: normalisation heads, image/prompt preparation, action queue."""

    config_class = PI05Config
    name = "pi05"
    model_class = PI05FlowMatching

    @staticmethod
    def _vocab_size(config) -> int:
        return gemma_2b_config(**(config.vlm or {})).vocab_size

    def __init__(self, config: PI05Config, per_dataset_stats: list[dict] | None = None,
                 dataset_names: list[str] | None = None, **_):
        super().__init__(config)
        config.validate_features()
        n_heads = (len(per_dataset_stats) if per_dataset_stats is not None
                   else len(config.dataset_names) if config.dataset_names else 1)
        kw = dict(per_dataset_stats=per_dataset_stats, dataset_names=dataset_names or config.dataset_names,
                  num_datasets=None if per_dataset_stats is not None else n_heads,
                  zero_range_center=config.zero_range_centers_on_zero, eps=config.normalization_epsilon)
        from ...configs.types import NormalizationMode
        self.normalize_inputs = Normalize(config.input_features, config.normalization_mapping, **kw)
        self.normalize_targets = Normalize(config.output_features, config.normalization_mapping, **kw)
        da_map = {"ACTION": NormalizationMode.MIN_MAX}
        self.normalize_discrete_actions = Normalize(config.output_features, da_map, **kw)
        self.unnormalize_outputs = Unnormalize(config.output_features, config.normalization_mapping, **kw)
        self.language_tokenizer = load_text_tokenizer(config.tokenizer_path, self._vocab_size(config))
        self.discrete_action_processor = load_action_tokenizer(config.discrete_action_tokenizer_path,
                                                               config.discrete_action_vocab_size)
        # a tokenizer fitted under the other zero-range convention would tokenize padded columns off its corpus
        self._check_discrete_action_tokenizer_convention(config.discrete_action_tokenizer_path)
        self.model = self.model_class(config, tokenizer=self.language_tokenizer)
        from ..utils import apply_policy_level_freezes
        apply_policy_level_freezes(self.model, self.model.wrapper, config)
        # uncertainty proxy and best-of-N are off until accel.configure_accel / candidates.configure_candidates
        # arm them; the attributes exist so that those switches can tell a wired sampler from an unwired one
        self.accel_prefix: int | None = None
        self.last_accel_provenance = None
        self.last_candidate_scores = None
        self._n_candidates, self._critic = 1, None
        self.reset()

    def reset(self) -> None:
        self._action_queue: deque = deque([], maxlen=self.config.n_action_steps)
        self.last_accel = None
        self.last_accel_candidates = None

    def get_optim_params(self):
        return [p for p in self.parameters() if p.requires_grad]

    def _prefix_kwargs(self, batch, normalized_batch) -> dict | None:
        """Extra prefix inputs of richer policies (state history, metadata, subgoals); none here."""
        return None

    # -- batch preparation ---------------------------------------------------------------------------
    def prepare_images(self, batch: dict[str, Any]) -> tuple[list[Tensor], list[Tensor]]:
        """Resize-with-pad to the model resolution, scale [0,1] -> [-1,1]; absent cameras become -1
        images with mask 0 (``modeling_pi05.py:1083-1141``)."""
        cfg = self.config
        keys = [k for k in cfg.image_features if not k.startswith("empty_camera")] or \
               sorted(k for k in batch if k.startswith("camera") and isinstance(batch[k], Tensor))
        present = [k for k in keys if k in batch]
        if not present:
            raise ValueError(f"all image features are missing from the batch (expected {keys})")
        images, masks = [], []
        pad_flags = batch.get("img_is_pad")
        for i, k in enumerate(present):
            img = batch[k]
            if img.dim() == 5:
                img = img[:, -1]
            if cfg.resize_imgs_with_padding is not None and tuple(img.shape[-2:]) != tuple(cfg.resize_imgs_with_padding):
                img = ops.resize_with_pad(img.float(), cfg.resize_imgs_with_padding[1],
                                          cfg.resize_imgs_with_padding[0], pad_value=0.0)
            img = img * 2.0 - 1.0
            B = img.shape[0]
            if pad_flags is not None:
                m = ~pad_flags[:, i].bool()
            else:
                m = torch.ones(B, dtype=torch.bool, device=img.device)
            images.append(img), masks.append(m)
        for _ in range(cfg.empty_cameras):
            images.append(torch.full_like(images[-1], -1.0))
            masks.append(torch.zeros_like(masks[-1]))
        return images, masks

    def prepare_discrete_state(self, batch) -> list[str]:
        state = batch["state"]
        if state.dim() == 3:
            state = state[:, -1]
        bins = torch.linspace(-1, 1, 257, device=state.device)[:-1]
        ids = (torch.bucketize(state.float().clamp(-1.0, 1.0), bins, right=True) - 1).clamp(0, 255)
        return [" ".join(map(str, row)) for row in ids.cpu().tolist()]

    def prepare_language(self, batch) -> tuple[Tensor, Tensor]:
        """Tokenises ``"Task: {task}, State: {bins};\\n"`` (discrete) or ``"Task: {task}, "`` (continuous state)
        (reference ``src/opentau/policies/pi05/modeling_pi05.py:1142-1180``);
        a batch that already carries ``lang_tokens``/``lang_masks`` is passed through."""
        cfg = self.config
        device = batch["state"].device
        if "lang_tokens" in batch:
            return batch["lang_tokens"].to(device), batch["lang_masks"].to(device).bool()
        tasks = batch["prompt"]
        if isinstance(tasks, str):
            tasks = [tasks]
        if cfg.state_type == "discrete":
            states = self.prepare_discrete_state(batch)
            prompts = [f"Task: {t}, State: {s};\n" for t, s in zip(tasks, states)]
        else:
            prompts = [f"Task: {t}, " for t in tasks]      # the state follows as its own "State: " block of the prefix
        enc = self.language_tokenizer(prompts, padding="max_length", padding_side="right",
                                      max_length=cfg.prompt_max_length, return_tensors="pt", truncation=True)
        return enc["input_ids"].to(device), enc["attention_mask"].to(device).bool()

    def prepare_response(self, batch) -> tuple[Tensor | None, Tensor | None]:
        cfg = self.config
        if not cfg.predict_response:
            return None, None
        device = batch["state"].device
        if "response_tokens" in batch:
            return batch["response_tokens"].to(device), batch["response_masks"].to(device).bool()
        resp = batch.get("response")
        if resp is None:
            return None, None
        enc = self.language_tokenizer([f"{r}" for r in resp], padding="max_length", padding_side="right",
                                      max_length=cfg.response_max_length, return_tensors="pt", truncation=True)
        return enc["input_ids"].to(device), enc["attention_mask"].to(device).bool()

    def prepare_discrete_actions(self, batch, norm_actions: Tensor) -> tuple[Tensor, Tensor]:
        cfg = self.config
        device = norm_actions.device
        if "discrete_actions" in batch:
            return batch["discrete_actions"].to(device), batch["discrete_action_masks"].to(device).bool()
        rows = self.discrete_action_processor(norm_actions.float().cpu())
        ids, mask = pad_tokens(rows, cfg.discrete_action_max_length)
        return ids.to(device), mask.to(device)

    # -- training / inference -----------------------------------------------------------------------
    def forward(self, batch: dict[str, Any], noise=None, time=None, return_per_sample: bool = False):
        B = batch["state"].shape[0]
        device = batch["state"].device
        idx = self._resolve_dataset_index(batch, B, device)
        nb = self.normalize_inputs(batch, idx)
        tb = self.normalize_targets(batch, idx)
        images, img_masks = self.prepare_images(nb)
        lang_tokens, lang_masks = self.prepare_language(nb)
        resp_t, resp_m = self.prepare_response(batch)
        if "discrete_actions" in batch:
            da, dam = self.prepare_discrete_actions(batch, tb["actions"])
        else:
            db = self.normalize_discrete_actions(batch, idx)
            da, dam = self.prepare_discrete_actions(batch, db["actions"])
        state = nb["state"]
        if state.dim() == 3:
            state = state[:, -1]
        out = self.model(images, img_masks, lang_tokens, lang_masks, tb["actions"],
                         actions_is_pad=batch.get("action_is_pad"), response_tokens=resp_t, response_masks=resp_m,
                         noise=noise, time=time, discrete_actions=da, discrete_action_masks=dam,
                         state=state if self.config.state_type == "continuous" else None,
                         real_action_dim=batch.get("real_action_dim"), return_per_sample=return_per_sample,
                         prefix_kwargs=self._prefix_kwargs(batch, nb))
        threshold = getattr(self.config, "warn_outlier_threshold", None)
        if threshold is not None and threshold > 0 and isinstance(out, dict):
            # Debug aid of the policies that carry the setting (reference pi07 low level ``forward``,
            # ``modeling_pi07_low_level.py:1003-1006``): pure and collective-free here; the trainer gathers and logs.
            from ..outlier_utils import detect_state_action_outliers
            probe = dict(batch)
            probe["state"], probe["actions"] = nb["state"], tb["actions"]
            out["outlier_records"] = detect_state_action_outliers(probe, threshold)
        return out

    @torch.no_grad()
    def sample_actions(self, batch: dict[str, Any], noise: Tensor | None = None, action_prefix: Tensor | None = None,
                       delay: int | Tensor = 0, n_candidates: int | None = None) -> Tensor:
        """Returns an un-normalised action chunk ``(B, chunk, real_dim)``.

        With ``n_candidates > 1`` (armed by ``candidates.configure_candidates`` or passed here) the expert denoises
        that many noise draws per observation over one prefix pass and the attached critic keeps one, scored in raw
        units on the executed rows (reference ``src/opentau/policies/pi05/modeling_pi05.py:780-867``).  With
        ``accel_prefix`` set, ``last_accel`` / ``last_accel_provenance`` are published for the emitted chunk."""
        from ..accel import make_meter, publish
        from ..candidates import expand_candidates, pick, select_candidate, warn_if_no_candidate_scored
        self.eval()
        cfg = self.config
        raw_state = self._delta_anchor_state(batch)          # before normalize_inputs: the raw state anchors the chunk
        B = batch["state"].shape[0]
        device = batch["state"].device
        idx = self._resolve_dataset_index(batch, B, device)
        nb = self.normalize_inputs(batch, idx)
        images, img_masks = self.prepare_images(nb)
        lang_tokens, lang_masks = self.prepare_language(nb)
        state = nb["state"]
        if state.dim() == 3:
            state = state[:, -1]
        if action_prefix is not None:
            action_prefix = self._model_space_prefix(action_prefix, raw_state, idx)
        n = int(n_candidates or getattr(self, "_n_candidates", None) or 1)
        critic = getattr(self, "_critic", None)
        if n > 1 and critic is None:
            from ..candidates import MEDOID, MedoidCritic
            if getattr(cfg, "action_chunk_critic_path", None) in (None, MEDOID):
                critic = MedoidCritic(self.unnormalize_outputs, max_action_dim=cfg.max_action_dim)
            else:
                raise ValueError(f"n_candidates={n} but no action-chunk critic is attached; arm best-of-N through "
                                 "candidates.configure_candidates")
        sampler_idx = expand_candidates(idx, n)
        meter = make_meter(self, batch_size=B * n, device=device, dataset_index=sampler_idx)
        st = state if cfg.state_type == "continuous" else None
        # the meter keeps host-side step counts, which a replayed graph would not advance: metered calls run eagerly
        if getattr(self, "_use_graphs", False) and device.type == "cuda" and meter is None and not cfg.predict_response:
            actions = self._graphed_sample(images, img_masks, lang_tokens, lang_masks, action_prefix, delay, noise,
                                           st, n)
        else:
            actions = self.model.sample_actions(images, img_masks, lang_tokens, lang_masks,
                                                action_prefix=action_prefix, delay=delay, noise=noise, state=st,
                                                n_candidates=n, accel=meter,
                                                prefix_kwargs=self._prefix_kwargs(batch, nb))
        self.last_response = self._decode_response()
        if n == 1:
            # before the un-normalisation: if that raises (non-finite buffers) the score is still there
            publish(self, meter, dataset_index=idx)
        feat = cfg.action_feature
        real = feat.shape[0] if feat is not None else actions.shape[-1]
        actions = self.unnormalize_outputs({"actions": actions[:, :, :real]}, sampler_idx)["actions"]
        if raw_state is not None:
            # the dataset subtracted the chunk-start state from the mapped dims; without the other half the consumer
            # would read displacements as absolute joint targets
            actions = add_chunk_start_state(actions, expand_candidates(raw_state, n).to(actions.dtype),
                                            cfg.delta_action_state_map)
        if n == 1:
            return actions
        candidates = actions.view(B, n, *actions.shape[1:])
        rows = self.model.executed_rows(delay, B, device)
        scores = critic.score_chunks(batch, candidates, row_mask=rows, dataset_index=idx)
        selected = select_candidate(scores)
        self.last_candidate_scores = scores.detach().to(torch.float32).cpu().tolist()
        warn_if_no_candidate_scored(self.last_candidate_scores)
        publish(self, meter, dataset_index=sampler_idx, n_candidates=n, selected=selected)
        return pick(candidates, selected)

    def _decode_response(self) -> list[str] | None:
        """The text the backbone generated for the last chunk (one string per observation), ``None`` when the policy
        does not predict responses; servers and planners read it from ``last_response``."""
        toks = getattr(self.model, "last_response_tokens", None)
        if toks is None:
            return None
        masks = self.model.last_response_masks
        rows = [t[m].tolist() for t, m in zip(toks.cpu(), masks.cpu())]
        return [self.language_tokenizer.decode(r, skip_special_tokens=True) for r in rows]

    def _delta_anchor_state(self, batch: dict[str, Any]) -> Tensor | None:
        """The RAW (un-normalised) state the emitted chunk is anchored to, when the policy was trained on delta joint
        actions; ``None`` for absolute actions.  A configured map without a ``state`` in the batch is an error: the
        inverse is impossible and returning displacements would silently emit actions in the wrong space
        (reference ``src/opentau/policies/pi05/modeling_pi05.py:896-927``)."""
        if not getattr(self.config, "delta_action_state_map", None):
            return None
        if "state" not in batch:
            raise KeyError("delta_action_state_map is configured, so sample_actions must add the conditioning state back "
                           f"onto its output, but the batch has no 'state' (keys: {sorted(batch)})")
        st = batch["state"].detach().clone().float()
        return st[:, -1] if st.dim() == 3 else st

    def _model_space_prefix(self, action_prefix: Tensor, raw_state: Tensor | None, idx: Tensor) -> Tensor:
        """The frozen rows of real-time chunking arrive as the caller holds them: ABSOLUTE, un-normalised actions off the
        queue.  The model was trained on (delta-transformed and) normalised targets, so the prefix takes the same route
        as a training target and is then padded to ``(B, chunk_size, max_action_dim)``."""
        cfg = self.config
        feat = cfg.action_feature
        real = min(feat.shape[0] if feat is not None else action_prefix.shape[-1], action_prefix.shape[-1])
        p = action_prefix[..., :real].float()
        if raw_state is not None:
            p = subtract_chunk_start_state(p, raw_state, cfg.delta_action_state_map)
        p = self.normalize_targets({"actions": p}, idx)["actions"]
        out = torch.zeros(p.shape[0], cfg.chunk_size, cfg.max_action_dim, dtype=torch.float32, device=p.device)
        out[:, :min(p.shape[1], cfg.chunk_size), :real] = p[:, :cfg.chunk_size]
        return out

    def enable_cuda_graphs(self, flag: bool = True) -> None:
        """Replay the sampler (prefix pass + Euler loop) from a CUDA graph: one launch per action chunk."""
        self._use_graphs = bool(flag)
        self._graph_runner = None

    def _graphed_sample(self, images, img_masks, lang_tokens, lang_masks, action_prefix, delay, noise, state, n):
        from ...runtime.graphs import CudaGraphRunner
        cfg = self.config
        B = lang_tokens.shape[0]
        device = lang_tokens.device
        if noise is None:
            noise = self.model.sample_noise((B * n, cfg.chunk_size, cfg.max_action_dim), device)
        if action_prefix is None:
            action_prefix = torch.zeros(B, cfg.chunk_size, cfg.max_action_dim, device=device)
        frozen = self.model.frozen_mask(delay, B, device).contiguous()
        has_state = state is not None
        if getattr(self, "_graph_runner", None) is None:
            def fn(images, img_masks, lang_tokens, lang_masks, noise, action_prefix, frozen, state):
                return self.model.sample_actions(list(images), list(img_masks), lang_tokens, lang_masks,
                                                 action_prefix=action_prefix, noise=noise, frozen=frozen,
                                                 state=state if has_state else None, n_candidates=n)
            self._graph_runner = CudaGraphRunner(fn)
        st = state if has_state else torch.zeros(1, device=device)
        out = self._graph_runner(tuple(images), tuple(img_masks), lang_tokens, lang_masks.bool(), noise.float(),
                                 action_prefix.float(), frozen, st)
        return out.clone()

    @torch.no_grad()
    def select_action(self, batch: dict[str, Any], noise: Tensor | None = None) -> Tensor:
        """Pops one action; refills the queue with a new chunk when it runs low
        (real-time chunking: the tail of the old chunk is the frozen prefix of the new one)."""
        cfg = self.config
        if len(self._action_queue) <= cfg.max_delay:
            prefix = None
            delay = len(self._action_queue)
            if delay > 0:
                tail = torch.stack(list(self._action_queue), dim=1)
                prefix = torch.zeros(tail.shape[0], cfg.chunk_size, cfg.max_action_dim, device=tail.device)
                prefix[:, :delay, :tail.shape[-1]] = tail
            actions = self.sample_actions(batch, noise=noise, action_prefix=prefix, delay=delay)
            self._action_queue.clear()
            self._action_queue.extend(actions.transpose(0, 1)[:cfg.n_action_steps])
        return self._action_queue.popleft()
