"""Gemma-3 backbone + Gemma-v1 action expert sharing attention (pi0.6 / pi0.7).

Module names mirror the reference wrapper so checkpoints interchange (OpenTau
``src/opentau/policies/pi07/gemma3_with_expert.py:349-722``):
``gemma3.model.{vision_tower, multi_modal_projector, language_model.{embed_tokens, norm}}``,
``gemma_expert.model.norm``, ``interleaved_layers.N.{backbone_layer, expert_layer}``,
``discrete_action_embedding``, ``da_head``.  One interleaved layer is the unit of sharding and of
activation checkpointing.  Backbone stream: q/k RMS-norm before RoPE, sandwich norms, per-layer RoPE base
(1e4 on sliding layers, 1e6 on global ones — also used by the expert stream of that layer), softmax scale
``query_pre_attn_scalar ** -0.5``; the sliding-window mask is never applied.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
from torch import Tensor, nn

from .. import ops
from .dual_stream import DualStreamDecoder
from .layers import DecoderLayer, Linear, TowerConfig, make_norm
from .siglip import Gemma3Projector, SiglipConfig, SiglipVisionModel


def gemma3_4b_config(**over) -> TowerConfig:
    return TowerConfig(**{**dict(hidden_size=2560, num_hidden_layers=34, num_attention_heads=8,
                                 num_key_value_heads=4, head_dim=256, intermediate_size=10240, vocab_size=262208,
                                 hidden_act="gelu_tanh", rope_theta=1_000_000.0, rope_local_theta=10_000.0,
                                 sliding_window_pattern=6, qk_norm=True, sandwich_norms=True,
                                 query_pre_attn_scalar=256.0), **over})


def gemma_expert_860m_config(**over) -> TowerConfig:
    return TowerConfig(**{**dict(hidden_size=1280, num_hidden_layers=34, num_attention_heads=8,
                                 num_key_value_heads=4, head_dim=256, intermediate_size=5120, vocab_size=262208,
                                 hidden_act="gelu_tanh", use_adarms=True, adarms_cond_dim=1280), **over})


class _TowerView:
    """What the shared decoder needs from a tower, assembled from the interleaved layers."""

    def __init__(self, cfg: TowerConfig, layers: list, norm: nn.Module):
        self.cfg, self.layers, self.norm = cfg, layers, norm


class InterleavedDecoderLayer(nn.Module):
    def __init__(self, backbone_layer: DecoderLayer, expert_layer: DecoderLayer | None):
        super().__init__()
        self.backbone_layer = backbone_layer
        if expert_layer is not None:
            self.expert_layer = expert_layer


class _LanguageModel(nn.Module):
    def __init__(self, cfg: TowerConfig):
        super().__init__()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        nn.init.normal_(self.embed_tokens.weight, std=0.02)
        self.norm = make_norm(cfg)


class _Gemma3Model(nn.Module):
    def __init__(self, text: TowerConfig, vision: SiglipConfig, tokens_per_side: int):
        super().__init__()
        self.vision_tower = SiglipVisionModel(vision)
        side = vision.image_size // vision.patch_size
        self.multi_modal_projector = Gemma3Projector(vision.hidden_size, text.hidden_size, side, tokens_per_side)
        self.language_model = _LanguageModel(text)


class _Gemma3(nn.Module):
    def __init__(self, text: TowerConfig, vision: SiglipConfig, tokens_per_side: int):
        super().__init__()
        self.model = _Gemma3Model(text, vision, tokens_per_side)


class _ExpertModel(nn.Module):
    def __init__(self, cfg: TowerConfig):
        super().__init__()
        self.norm = make_norm(cfg)


class _GemmaExpert(nn.Module):
    def __init__(self, cfg: TowerConfig):
        super().__init__()
        self.model = _ExpertModel(cfg)


@dataclass
class Gemma3WithExpertConfig:
    text: dict = field(default_factory=dict)
    expert: dict = field(default_factory=dict)
    vision: dict = field(default_factory=dict)
    image_size: int = 448
    tokens_per_image_side: int = 16
    freeze_vision_encoder: bool = True
    train_expert_only: bool = False
    train_vision_encoder_only: bool = False
    train_state_action_representation_only: bool = False
    discrete_action_vocab_size: int = 2048
    dropout: float = 0.1
    gradient_checkpointing: bool = False
    disable_action_expert: bool = False


class Gemma3WithExpertModel(nn.Module):
    def __init__(self, config: Gemma3WithExpertConfig):
        super().__init__()
        self.config = config
        text = gemma3_4b_config(**config.text)
        exp_over = dict(config.expert)
        exp_over.setdefault("num_hidden_layers", text.num_hidden_layers)
        expert = gemma_expert_860m_config(**exp_over)
        if "hidden_size" in exp_over and "adarms_cond_dim" not in exp_over:
            expert.adarms_cond_dim = expert.hidden_size
        vision = SiglipConfig(**{**dict(image_size=config.image_size), **config.vision})
        self.vlm_cfg, self.expert_cfg, self.vision_cfg = text, expert, vision
        self.gemma3 = _Gemma3(text, vision, config.tokens_per_image_side)
        self.gemma_expert = None if config.disable_action_expert else _GemmaExpert(expert)
        self.discrete_action_embedding = nn.Embedding(config.discrete_action_vocab_size, text.hidden_size,
                                                      padding_idx=0)
        self.da_head = Linear(text.hidden_size, config.discrete_action_vocab_size, bias=True)
        self.interleaved_layers = nn.ModuleList([
            InterleavedDecoderLayer(DecoderLayer(text, i),
                                    None if config.disable_action_expert else DecoderLayer(expert, i))
            for i in range(text.num_hidden_layers)])
        towers = [_TowerView(text, [l.backbone_layer for l in self.interleaved_layers],
                             self.gemma3.model.language_model.norm)]
        if self.gemma_expert is not None:
            towers.append(_TowerView(expert, [l.expert_layer for l in self.interleaved_layers],
                                     self.gemma_expert.model.norm))
        self.decoder = DualStreamDecoder(towers, dropout=config.dropout,
                                         gradient_checkpointing=config.gradient_checkpointing)
        self.set_requires_grad()

    def set_requires_grad(self) -> None:
        c = self.config
        vt = self.gemma3.model.vision_tower
        if c.freeze_vision_encoder:
            vt.eval()
            for p in vt.parameters():
                p.requires_grad = False
        if c.train_expert_only:
            for p in self.gemma3.parameters():
                p.requires_grad = False
            for l in self.interleaved_layers:
                for p in l.backbone_layer.parameters():
                    p.requires_grad = False
        if c.train_vision_encoder_only:
            for p in self.parameters():
                p.requires_grad = False
            for p in list(vt.parameters()) + list(self.gemma3.model.multi_modal_projector.parameters()):
                p.requires_grad = True
        if c.train_state_action_representation_only:
            for p in self.parameters():
                p.requires_grad = False
            for p in list(self.discrete_action_embedding.parameters()) + list(self.da_head.parameters()):
                p.requires_grad = True

    def train(self, mode: bool = True):
        super().train(mode)
        if self.config.freeze_vision_encoder:
            self.gemma3.model.vision_tower.eval()
        return self

    def embed_image(self, image: Tensor) -> Tensor:
        feats = self.gemma3.model.vision_tower(image)
        return self.gemma3.model.multi_modal_projector(feats)

    def embed_language_tokens(self, tokens: Tensor) -> Tensor:
        """Gemma-3 token embeddings are scaled by ``sqrt(hidden)`` inside the embedding layer."""
        return ops.embedding(self.gemma3.model.language_model.embed_tokens.weight, tokens,
                             math.sqrt(self.vlm_cfg.hidden_size))

    def embed_discrete_actions(self, actions: Tensor) -> Tensor:
        return ops.embedding(self.discrete_action_embedding.weight, actions, padding_idx=0)

    def lm_head_weight(self) -> Tensor:
        return self.gemma3.model.language_model.embed_tokens.weight

    def forward(self, inputs_embeds, position_ids, q_blk, q_valid, **kw):
        if len(self.decoder.towers) == 1:
            outs, cache = self.decoder([inputs_embeds[0]], position_ids, q_blk, q_valid, **{
                k: ([v[0]] if k == "adarms_cond" and v is not None else v) for k, v in kw.items()})
            return [outs[0], None], cache
        return self.decoder(inputs_embeds, position_ids, q_blk, q_valid, **kw)
