"""Value model: SigLIP images + Gemma-3 270M text -> a categorical distribution over return bins.

Sequence (reference ``src/opentau/policies/value/modeling_value.py:645-869`` and
``value/siglip_gemma.py:142-291``):

    image tokens (bidirectional) | prompt "Task: ..<eos>State: ..<eos>" (bidirectional with the images) |
    [VALUE] learned token (opens a causal block) | response tokens (causal, training only)

The hidden state at the value token goes through ``value_head`` (``number_of_bins`` classes over the
normalised return range [-1, 0]); the response positions are trained with next-token CE so that language
co-training data (samples whose actions are all padding) shares the backbone.  The expected value is the
softmax-weighted mean of the bin centres.

The backbone is a single-tower pass through the shared two-stream decoder (q/k-norm, sandwich norms,
per-layer RoPE base), so every matrix product, norm and the block-causal attention are the sm_100a kernels;
the response head never materialises ``(B*L, vocab)`` logits (fused linear + cross-entropy).

State-dict keys follow the reference: ``model.siglip_gemma_value.{vision_encoder, gemma, value_head,
value_token, response_head}``, ``model.state_proj``, ``model.multi_modal_proj``.
"""

from __future__ import annotations

import math
from typing import Any

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from ... import ops
from ...models.dual_stream import DualStreamDecoder
from ...models.layers import Linear, Tower, TowerConfig
from ...models.siglip import SiglipConfig, SiglipVisionModel
from ...utils.tokenizer import load_text_tokenizer
from ..normalize import Normalize
from ..pretrained import PreTrainedPolicy
from ..utils import PerSampleLoss, ce_per_sample
from .configuration_value import ValueConfig


def gemma3_270m_config(**over) -> TowerConfig:
    return TowerConfig(**{**dict(hidden_size=640, num_hidden_layers=18, num_attention_heads=4,
                                 num_key_value_heads=1, head_dim=256, intermediate_size=2048, vocab_size=262144,
                                 hidden_act="gelu_tanh", rope_theta=1_000_000.0, rope_local_theta=10_000.0,
                                 sliding_window_pattern=6, qk_norm=True, sandwich_norms=True,
                                 query_pre_attn_scalar=256.0), **over})


class SiglipGemmaValueModel(nn.Module):
    """Vision encoder, text decoder, the value token and the two heads."""

    def __init__(self, text: TowerConfig, vision: SiglipConfig, num_value_bins: int, response_max_length: int):
        super().__init__()
        self.text_cfg, self.vision_cfg = text, vision
        self.response_max_length = response_max_length
        self.vision_encoder = SiglipVisionModel(vision)
        self.gemma = Tower(text)
        self.value_head = Linear(text.hidden_size, num_value_bins, bias=True)
        self.value_token = nn.Parameter(torch.zeros(1, 1, text.hidden_size))
        nn.init.normal_(self.value_token, std=0.02)
        self.response_head = Linear(text.hidden_size, text.vocab_size, bias=False)
        self.decoder = DualStreamDecoder([self.gemma])

    def embed_image(self, image: Tensor) -> Tensor:
        return self.vision_encoder(image)

    def embed_language_tokens(self, tokens: Tensor) -> Tensor:
        return self.gemma.embed(tokens)

    def hidden(self, inputs_embeds: Tensor, position_ids: Tensor, q_blk: Tensor, q_valid: Tensor) -> Tensor:
        (h,), _ = self.decoder([inputs_embeds], position_ids, q_blk, q_valid)
        return h

    def forward(self, inputs_embeds, position_ids, q_blk, q_valid) -> tuple[Tensor, Tensor]:
        """``(value_logits (B, bins), response_hidden (B, R-1, d))`` for a sequence that ends in R response tokens."""
        h = self.hidden(inputs_embeds, position_ids, q_blk, q_valid)
        R = self.response_max_length
        return self.value_head(h[:, -R - 1]), h[:, -R:-1]

    def get_value(self, inputs_embeds, position_ids, q_blk, q_valid) -> Tensor:
        """Value logits when the sequence ends at the value token (inference, no response)."""
        h = self.hidden(inputs_embeds, position_ids, q_blk, q_valid)
        return self.value_head(h[:, -1])


class ValueModel(nn.Module):
    def __init__(self, config: ValueConfig):
        super().__init__()
        self.config = config
        text = gemma3_270m_config(**(config.vlm or {}))
        vision = SiglipConfig(**{**dict(image_size=config.resize_imgs_with_padding[0]), **(config.vision or {})})
        self.siglip_gemma_value = SiglipGemmaValueModel(text, vision, config.reward_config.number_of_bins,
                                                        config.response_max_length)
        self.state_proj = Linear(config.max_state_dim, text.hidden_size, bias=True)
        self.multi_modal_proj = Linear(vision.hidden_size, text.hidden_size, bias=True)
        self.bins = config.reward_config.number_of_bins
        self.c_neg = config.reward_config.C_neg

    def embed_sequence(self, images, img_masks, lang_tokens, lang_masks, response_tokens=None, response_masks=None):
        """Returns ``(embeddings, pad_mask, block_ids)``; block ids encode the attention pattern directly."""
        m = self.siglip_gemma_value
        dtype = self.multi_modal_proj.weight.dtype
        B = lang_tokens.shape[0]
        device = lang_tokens.device
        embs, pads = [], []
        stacked = torch.stack(images, dim=1).flatten(0, 1)           # all cameras in one tower pass
        img = self.multi_modal_proj(m.embed_image(stacked).to(dtype))
        n_img = img.shape[1]
        embs.append(img.view(B, len(images) * n_img, -1))
        pads.append(torch.stack(img_masks, dim=1)[:, :, None].expand(B, len(images), n_img).reshape(B, -1))
        embs.append(m.embed_language_tokens(lang_tokens).to(dtype))
        pads.append(lang_masks.bool())
        n_bidir = embs[0].shape[1] + embs[1].shape[1]
        embs.append(m.value_token.to(dtype).expand(B, 1, -1))
        pads.append(torch.ones(B, 1, dtype=torch.bool, device=device))
        n_causal = 1
        if response_tokens is not None:
            r = m.embed_language_tokens(response_tokens).to(dtype)
            # the reference scales the (already scaled) response embeddings by sqrt(d) once more
            embs.append(r * math.sqrt(r.shape[-1]))
            pads.append(response_masks.bool())
            n_causal += r.shape[1]
        x = torch.cat(embs, dim=1)
        pad = torch.cat(pads, dim=1)
        blk = torch.cat([torch.zeros(n_bidir, dtype=torch.int32, device=device),
                         torch.arange(1, n_causal + 1, dtype=torch.int32, device=device)])[None].expand(B, -1)
        return x, pad, blk

    def _run(self, fn, images, img_masks, lang_tokens, lang_masks, response_tokens=None, response_masks=None):
        x, pad, blk = self.embed_sequence(images, img_masks, lang_tokens, lang_masks, response_tokens, response_masks)
        pos = torch.cumsum(pad, dim=1) - 1
        return fn(x, pos, blk.contiguous(), pad)

    def forward(self, images, img_masks, lang_tokens, lang_masks, response_tokens, response_masks):
        return self._run(self.siglip_gemma_value, images, img_masks, lang_tokens, lang_masks, response_tokens,
                         response_masks)

    def get_value(self, images, img_masks, lang_tokens, lang_masks) -> Tensor:
        return self._run(self.siglip_gemma_value.get_value, images, img_masks, lang_tokens, lang_masks)


class ValueFunction(PreTrainedPolicy):
    """Policy-API wrapper: ``forward`` = training losses, ``predict_value`` = expected normalised return."""

    config_class = ValueConfig
    name = "value"

    def __init__(self, config: ValueConfig, per_dataset_stats: list[dict] | None = None,
                 dataset_names: list[str] | None = None, **_):
        super().__init__(config)
        config.validate_features()
        n_heads = (len(per_dataset_stats) if per_dataset_stats is not None
                   else len(config.dataset_names) if config.dataset_names else 1)
        self.normalize_inputs = Normalize(
            config.input_features, config.normalization_mapping, per_dataset_stats=per_dataset_stats,
            dataset_names=dataset_names or config.dataset_names,
            num_datasets=None if per_dataset_stats is not None else n_heads,
            zero_range_center=config.zero_range_centers_on_zero, eps=config.normalization_epsilon)
        self.language_tokenizer = load_text_tokenizer(
            config.tokenizer_path, gemma3_270m_config(**(config.vlm or {})).vocab_size)
        self.model = ValueModel(config)

    def reset(self) -> None:
        pass

    def get_optim_params(self):
        return [p for p in self.parameters() if p.requires_grad]

    # -- value read-out ----------------------------------------------------------------------------
    def bin_centres(self, device) -> Tensor:
        n = self.config.reward_config.number_of_bins
        lo = torch.linspace(-1, -1 / n, n, device=device)
        hi = torch.linspace(-1 + 1 / n, 0, n, device=device)
        return (lo + hi) / 2

    def calculate_value(self, logits: Tensor) -> Tensor:
        """Expected normalised return ``(B,)`` under the predicted bin distribution."""
        return torch.softmax(logits.float(), dim=-1) @ self.bin_centres(logits.device)

    # -- batch preparation ---------------------------------------------------------------------------
    def prepare_images(self, batch) -> tuple[list[Tensor], list[Tensor]]:
        cfg = self.config
        keys = list(cfg.image_features)
        present = [k for k in keys if k in batch]
        missing = [k for k in keys if k not in batch]
        if not present:
            raise ValueError(f"All image features are missing from the batch. At least one expected. "
                             f"(batch: {list(batch)}) (image_features: {keys})")
        images, masks = [], []
        for k in present:
            img = batch[k]
            if cfg.resize_imgs_with_padding is not None and tuple(img.shape[-2:]) != tuple(cfg.resize_imgs_with_padding):
                img = ops.resize_with_pad(img.float(), cfg.resize_imgs_with_padding[1],
                                          cfg.resize_imgs_with_padding[0], pad_value=0.0)
            images.append(img * 2.0 - 1.0)
            masks.append(torch.ones(img.shape[0], dtype=torch.bool, device=img.device))
        for _ in range(min(len(missing), cfg.empty_cameras)):
            images.append(torch.full_like(images[-1], -1.0))
            masks.append(torch.zeros_like(masks[-1]))
        return images, masks

    def prepare_discrete_state(self, batch) -> list[str]:
        state = batch["state"].float().clamp(-1.0, 1.0)
        bins = torch.linspace(-1, 1, 257, device=state.device)[:-1]
        ids = torch.bucketize(state, bins, right=True) - 1
        return [" ".join(map(str, row)) for row in ids.cpu().tolist()]

    def prepare_language(self, batch) -> tuple[Tensor, Tensor]:
        device = batch["state"].device
        if "lang_tokens" in batch:
            return batch["lang_tokens"].to(device), batch["lang_masks"].to(device).bool()
        prompts = [f"Task: {t}<eos>State: {s}<eos>" for t, s in zip(batch["prompt"], self.prepare_discrete_state(batch))]
        enc = self.language_tokenizer(prompts, padding="max_length", padding_side="right",
                                      max_length=self.config.prompt_max_length, return_tensors="pt", truncation=True)
        return enc["input_ids"].to(device), enc["attention_mask"].to(device).bool()

    def prepare_response(self, batch) -> tuple[Tensor, Tensor]:
        device = batch["state"].device
        if "response_tokens" in batch:
            return batch["response_tokens"].to(device), batch["response_masks"].to(device).bool()
        resp = batch.get("response") or [""] * batch["state"].shape[0]
        enc = self.language_tokenizer([f"{r}" for r in resp], padding="max_length", padding_side="right",
                                      max_length=self.config.response_max_length, return_tensors="pt",
                                      truncation=True)
        return enc["input_ids"].to(device), enc["attention_mask"].to(device).bool()

    # -- API -----------------------------------------------------------------------------------------
    @torch.no_grad()
    def select_action(self, batch: dict[str, Tensor]) -> Tensor:
        raise NotImplementedError("Value functions do not select actions. Use predict_value() instead.")

    def sample_actions(self, batch: dict[str, Tensor], noise: Tensor | None = None):
        raise NotImplementedError("Value functions do not sample actions. Use predict_value() instead.")

    @torch.no_grad()
    def predict_value(self, batch: dict[str, Any]) -> Tensor:
        self.eval()
        B, device = batch["state"].shape[0], batch["state"].device
        nb = self.normalize_inputs(batch, self._resolve_dataset_index(batch, B, device))
        images, img_masks = self.prepare_images(nb)
        lang_tokens, lang_masks = self.prepare_language(nb)
        return self.calculate_value(self.model.get_value(images, img_masks, lang_tokens, lang_masks))

    def forward(self, batch: dict[str, Any], return_per_sample: bool = False) -> dict[str, Any]:
        """Losses: ``CE`` = value-bin CE on robot samples + response CE on language-only samples (those whose
        ``action_is_pad`` is all True); ``L1`` and ``Accuracy`` are monitors; ``MSE`` is a zero stub."""
        B, device = batch["state"].shape[0], batch["state"].device
        nb = self.normalize_inputs(batch, self._resolve_dataset_index(batch, B, device))
        images, img_masks = self.prepare_images(nb)
        lang_tokens, lang_masks = self.prepare_language(nb)
        resp_t, resp_m = self.prepare_response(batch)
        value_logits, resp_h = self.model(images, img_masks, lang_tokens, lang_masks, resp_t, resp_m)
        values = self.calculate_value(value_logits)
        value_logits = value_logits.float()
        target = batch["return_bin_idx"].long().view(B)
        pad = batch.get("action_is_pad")
        lang_only = pad.bool().all(dim=1) if pad is not None else torch.zeros(B, dtype=torch.bool, device=device)
        robot = (~lang_only).float()
        v_ce = F.cross_entropy(value_logits, target, reduction="none") * robot
        l1 = F.l1_loss(values, batch["return_continuous"].float().view(B))
        acc = ((value_logits.argmax(-1) == target).float() * robot).sum() / robot.sum().clamp(min=1)

        L = resp_h.shape[1]
        head = self.model.siglip_gemma_value.response_head
        r_ce = ops.linear_cross_entropy(resp_h.reshape(B * L, -1), head.weight, None,
                                        resp_t[:, 1:].reshape(-1)).view(B, L)
        r_valid = resp_m[:, 1:] & lang_only[:, None]
        r_ce = r_ce * r_valid.to(r_ce.dtype)
        out: dict[str, Any] = {"MSE": torch.zeros((), device=device), "CE": v_ce.mean() + r_ce.mean(),
                               "L1": l1, "Accuracy": acc}
        if return_per_sample:
            z = torch.zeros(B, device=device)
            out["MSE_per_sample"] = PerSampleLoss(z, z.clone())
            out["CE_per_sample"] = PerSampleLoss(v_ce, robot) + ce_per_sample(r_ce, r_valid)
        return out
