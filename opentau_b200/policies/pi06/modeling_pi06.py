"""pi0.6: Gemma-3-4B + SigLIP@448 (avg-pooled to 256 tokens per camera) + 860 M flow-matching expert.

Differences from pi0.5 (reference ``src/opentau/policies/pi06/modeling_pi06.py:970-1152``): language
tokens are causal (each opens a new attention block), the FAST block has no ``"Action: "`` indicator,
the backbone has q/k-norm, sandwich norms and per-layer RoPE bases, and sampling takes 5 Euler steps.
State-dict keys live under ``model.gemma3_with_expert.*``.
"""

from __future__ import annotations

import torch
from torch import Tensor

from ...models.gemma3_with_expert import Gemma3WithExpertConfig, Gemma3WithExpertModel, gemma3_4b_config
from ..pi05.modeling_pi05 import PI05FlowMatching, PI05Policy
from .configuration_pi06 import PI06Config


def wrapper_config_from(config) -> Gemma3WithExpertConfig:
    vc = dict(getattr(config, "vlm_config", None) or {})
    text = {**vc.get("text", {}), **(getattr(config, "vlm", None) or {})}
    expert = {**vc.get("expert", {}), **(getattr(config, "expert", None) or {})}
    vision = {**vc.get("vision", {}), **(getattr(config, "vision", None) or {})}
    return Gemma3WithExpertConfig(
        text=text, expert=expert, vision=vision, image_size=config.resize_imgs_with_padding[0],
        tokens_per_image_side=vc.get("tokens_per_image_side", 16),
        freeze_vision_encoder=config.freeze_vision_encoder, train_expert_only=config.train_expert_only,
        train_vision_encoder_only=config.train_vision_encoder_only,
        train_state_action_representation_only=config.train_state_action_representation_only,
        discrete_action_vocab_size=config.discrete_action_vocab_size, dropout=config.dropout,
        gradient_checkpointing=config.gradient_checkpointing,
        disable_action_expert=vc.get("disable_action_expert", False))


class PI06FlowMatching(PI05FlowMatching):
    wrapper_attr = "gemma3_with_expert"

    def build_wrapper(self, config):
        return Gemma3WithExpertModel(wrapper_config_from(config))

    def discrete_block_len(self) -> int:
        return self.config.discrete_action_max_length

    def embed_prefix(self, images, img_masks, lang_tokens, lang_masks, response_tokens=None, response_masks=None,
                     discrete_actions=None, discrete_action_masks=None, state=None):
        w = self.wrapper
        dtype = w.da_head.weight.dtype
        device = lang_tokens.device
        B = lang_tokens.shape[0]
        embs, pads, att = [], [], []
        if images:
            stacked = torch.stack(images, dim=1).flatten(0, 1)
            img_emb = w.embed_image(stacked).to(dtype)
            n_img = img_emb.shape[1]
            embs.append(img_emb.view(B, len(images) * n_img, -1))
            pads.append(torch.stack(img_masks, dim=1)[:, :, None].expand(B, len(images), n_img).reshape(B, -1))
            att += [0] * (len(images) * n_img)
        lang = w.embed_language_tokens(lang_tokens).to(dtype)
        embs.append(lang), pads.append(lang_masks.bool())
        att += [1] * lang.shape[1]                      # causal text
        if response_tokens is not None:
            r = w.embed_language_tokens(response_tokens).to(dtype)
            embs.append(r), pads.append(response_masks.bool())
            att += [1] * r.shape[1]
        if discrete_actions is not None:
            d = w.embed_discrete_actions(discrete_actions).to(dtype)
            embs.append(d), pads.append(discrete_action_masks.bool())
            att += [1] * d.shape[1]
        embs_t = torch.cat(embs, dim=1)
        pads_t = torch.cat(pads, dim=1)
        att_t = self._const(("att", tuple(att), str(device)),
                            lambda: torch.tensor(att, dtype=torch.bool, device=device))[None].expand(B, -1)
        return embs_t, pads_t, att_t, None


class PI06Policy(PI05Policy):
    config_class = PI06Config
    name = "pi06"
    model_class = PI06FlowMatching

    @staticmethod
    def _vocab_size(config) -> int:
        vc = dict(getattr(config, "vlm_config", None) or {})
        return gemma3_4b_config(**{**vc.get("text", {}), **(config.vlm or {})}).vocab_size

    def prepare_language(self, batch):
        """``"Task: {task}<eos>State: {bins}<eos>Response:"`` when the backbone predicts a response, else
        ``"...<eos>Actions:"``: the prefix has no separate indicator blocks, the prompt spells the separators out
        (reference ``src/opentau/policies/pi06/modeling_pi06.py:908-943``)."""
        device = batch["state"].device
        if "lang_tokens" in batch:
            return batch["lang_tokens"].to(device), batch["lang_masks"].to(device).bool()
        tasks = batch["prompt"]
        tasks = [tasks] if isinstance(tasks, str) else list(tasks)
        tail = "Response:" if self.config.predict_response else "Actions:"
        prompts = [f"Task: {t}<eos>State: {s}<eos>{tail}" for t, s in zip(tasks, self.prepare_discrete_state(batch))]
        enc = self.language_tokenizer(prompts, padding="max_length", padding_side="right",
                                      max_length=self.config.prompt_max_length, return_tensors="pt", truncation=True)
        return enc["input_ids"].to(device), enc["attention_mask"].to(device).bool()

    def prepare_response(self, batch):
        """``"{response}<eos>Actions:"``: the response closes with the separator and hands over to the action block."""
        cfg = self.config
        if not cfg.predict_response:
            return None, None
        device = batch["state"].device
        if "response_tokens" in batch:
            return batch["response_tokens"].to(device), batch["response_masks"].to(device).bool()
        resp = batch.get("response")
        if resp is None:
            return None, None
        enc = self.language_tokenizer([f"{r}<eos>Actions:" for r in resp], padding="max_length", padding_side="right",
                                      max_length=cfg.response_max_length, return_tensors="pt", truncation=True)
        return enc["input_ids"].to(device), enc["attention_mask"].to(device).bool()
