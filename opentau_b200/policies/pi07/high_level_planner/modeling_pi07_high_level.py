"""pi0.7 high-level planner: Gemma-3 VLM (no action expert) that writes an updated memory and the next subtask.

Prefix layout (reference ``src/opentau/policies/pi07/high_level_planner/modeling_pi07_high_level.py:992-1209``):

    images (bidirectional) | prompt (causal) | metadata? | ";\\n "? | "Updated Memory: " | memory |
    "Subtask: " | response

Training minimises next-token CE over the memory and response segments (``MSE`` is identically zero);
inference greedily decodes the memory, then the subtask, against a growing KV cache.
"""

from __future__ import annotations

from typing import Any

import torch
from torch import Tensor, nn

from .... import ops
from ....models.dual_stream import KVCache
from ....models.gemma3_with_expert import Gemma3WithExpertConfig, Gemma3WithExpertModel, gemma3_4b_config
from ....utils.tokenizer import load_text_tokenizer
from ...normalize import Normalize
from ...pretrained import PreTrainedPolicy
from ..common import global_or_branch_decisions
from .configuration_pi07_high_level import PI07HighLevelPlannerConfig


class PI07HighLevelPlannerModel(nn.Module):
    def __init__(self, config: PI07HighLevelPlannerConfig, tokenizer):
        super().__init__()
        self.config = config
        self.language_tokenizer = tokenizer
        setattr(self, self.wrapper_attr, self.build_wrapper(config))
        self.sync_branches = True
        self._ids: dict[str, list[int]] = {}

    wrapper_attr = "gemma3_with_expert"

    def build_wrapper(self, config):
        vc = dict(config.vlm_config or {})
        wcfg = Gemma3WithExpertConfig(
            text={**vc.get("text", {}), **(config.vlm or {})}, vision={**vc.get("vision", {}), **(config.vision or {})},
            image_size=config.resize_imgs_with_padding[0], tokens_per_image_side=vc.get("tokens_per_image_side", 16),
            freeze_vision_encoder=config.freeze_vision_encoder, dropout=config.dropout,
            gradient_checkpointing=config.gradient_checkpointing, disable_action_expert=True,
            discrete_action_vocab_size=8)
        return Gemma3WithExpertModel(wcfg)

    @property
    def wrapper(self):
        return getattr(self, self.wrapper_attr)

    def _indicator(self, text: str, B: int, device, max_len: int | None = None) -> tuple[Tensor, Tensor]:
        if text not in self._ids:
            self._ids[text] = list(self.language_tokenizer.encode(text, add_special_tokens=False))
        ids = self._ids[text]
        if max_len is not None:
            ids = (ids + [0] * max_len)[:max_len]
        tok = torch.tensor([ids], device=device).expand(B, -1)
        return tok, torch.ones(B, len(ids), dtype=torch.bool, device=device)

    def embed_context(self, images, img_masks, lang_tokens, lang_masks, metadata_tokens=None, metadata_masks=None):
        """Everything up to (excluding) the ``"Updated Memory: "`` indicator."""
        w = self.wrapper
        dtype = w.da_head.weight.dtype
        B, device = lang_tokens.shape[0], lang_tokens.device
        embs, pads, att = [], [], []
        if images:
            stacked = torch.stack(images, dim=1).flatten(0, 1)
            e = w.embed_image(stacked).to(dtype)
            n = e.shape[1]
            embs.append(e.view(B, len(images) * n, -1))
            pads.append(torch.stack(img_masks, 1)[:, :, None].expand(B, len(images), n).reshape(B, -1))
            att += [0] * (len(images) * n)
        embs.append(w.embed_language_tokens(lang_tokens).to(dtype)), pads.append(lang_masks.bool())
        att += [1] * lang_tokens.shape[1]
        present = (metadata_tokens is not None,)
        anys = (present[0] and bool(metadata_masks.any()),)
        (has_meta,) = global_or_branch_decisions(present, anys, ("metadata",), device, self.sync_branches)
        if has_meta and metadata_tokens is not None:
            embs.append(w.embed_language_tokens(metadata_tokens).to(dtype)), pads.append(metadata_masks.bool())
            att += [1] * metadata_tokens.shape[1]
            t, m = self._indicator(";\n ", B, device)
            embs.append(w.embed_language_tokens(t).to(dtype)), pads.append(m)
            att += [1] * t.shape[1]
        return torch.cat(embs, 1), torch.cat(pads, 1), att

    def forward(self, images, img_masks, lang_tokens, lang_masks, memory_tokens, memory_masks, response_tokens,
                response_masks, metadata_tokens=None, metadata_masks=None, return_per_sample=False):
        cfg, w = self.config, self.wrapper
        B, device = lang_tokens.shape[0], lang_tokens.device
        embs, pads, att = self.embed_context(images, img_masks, lang_tokens, lang_masks, metadata_tokens,
                                             metadata_masks)
        dtype = embs.dtype
        mi_t, mi_m = self._indicator("Updated Memory: ", B, device, cfg.memory_indicator_max_length)
        si_t, si_m = self._indicator("Subtask: ", B, device, cfg.subtask_indicator_max_length)
        segs = [(mi_t, mi_m), (memory_tokens, memory_masks.bool()), (si_t, si_m),
                (response_tokens, response_masks.bool())]
        tail_tokens = torch.cat([s[0] for s in segs], 1)
        tail_masks = torch.cat([s[1] for s in segs], 1)
        x = torch.cat([embs, w.embed_language_tokens(tail_tokens).to(dtype)], 1)
        pad = torch.cat([pads, tail_masks], 1)
        att_t = torch.tensor(att + [1] * tail_tokens.shape[1], dtype=torch.bool, device=device)[None].expand(B, -1)
        blk, valid = ops.make_block_ids(pad, att_t)
        pos = torch.cumsum(pad, 1) - 1
        (out, _), _ = w(inputs_embeds=[x, None], position_ids=pos, q_blk=blk, q_valid=valid)
        # next-token CE over the memory and the response segments (tail-relative slices)
        Lt = tail_tokens.shape[1]
        h = out[:, -Lt - 1:-1]
        labels = tail_tokens
        target_mask = torch.cat([torch.zeros_like(mi_m), memory_masks.bool(), torch.zeros_like(si_m),
                                 response_masks.bool()], 1)
        ce = ops.linear_cross_entropy(h.reshape(B * Lt, -1), w.lm_head_weight(), None, labels.reshape(-1)).view(B, Lt)
        ce = ce * target_mask.to(ce.dtype)
        loss = ce.sum() / target_mask.sum().clamp_min(1)
        res = {"MSE": torch.zeros((), device=device), "CE": loss}
        if return_per_sample:
            z = torch.zeros(B, device=device)
            res["MSE_per_sample"], res["CE_per_sample"] = (z, z.clone()), (ce.sum(1), target_mask.sum(1).float())
        return res

    @torch.no_grad()
    def _decode(self, cache: KVCache, next_pos: Tensor, first_tokens: Tensor, max_new: int, eos_id: int):
        """Feeds ``first_tokens`` then greedily extends by up to ``max_new`` tokens.  Returns (tokens, cache, pos)."""
        w = self.wrapper
        B, device = first_tokens.shape[0], first_tokens.device
        feed = first_tokens
        out_tokens = []
        done = torch.zeros(B, dtype=torch.bool, device=device)
        for step in range(max_new + 1):
            n = feed.shape[1]
            x = w.embed_language_tokens(feed).to(w.da_head.weight.dtype)
            pad = torch.ones(B, n, dtype=torch.bool, device=device)
            blk, valid = ops.make_block_ids(pad, pad)
            pos = next_pos[:, None] + torch.arange(n, device=device)[None]
            (h, _), new = w(inputs_embeds=[x, None], position_ids=pos, q_blk=blk, q_valid=valid, past=cache,
                            fill_cache_len=n)
            cache = KVCache(torch.cat([cache.k[:, :, :cache.length], new.k], 2),
                            torch.cat([cache.v[:, :, :cache.length], new.v], 2),
                            torch.cat([cache.valid[:, :cache.length], pad], 1), cache.length + n)
            next_pos = next_pos + n
            if step == max_new:
                break
            logits = ops.linear(h[:, -1], w.lm_head_weight()).float()
            tok = logits.argmax(-1)
            tok = torch.where(done, torch.zeros_like(tok), tok)
            out_tokens.append(tok)
            done |= tok == eos_id
            feed = tok[:, None]
        toks = torch.stack(out_tokens, 1) if out_tokens else torch.zeros(B, 0, dtype=torch.long, device=device)
        return toks, cache, next_pos

    @torch.no_grad()
    def generate(self, images, img_masks, lang_tokens, lang_masks, metadata_tokens=None, metadata_masks=None):
        """Two greedy decodes: memory (after ``"Updated Memory: "``) then subtask (after ``"Subtask: "``)."""
        cfg, w = self.config, self.wrapper
        B, device = lang_tokens.shape[0], lang_tokens.device
        embs, pads, att = self.embed_context(images, img_masks, lang_tokens, lang_masks, metadata_tokens,
                                             metadata_masks)
        att_t = torch.tensor(att, dtype=torch.bool, device=device)[None].expand(B, -1)
        blk, valid = ops.make_block_ids(pads, att_t)
        pos = torch.cumsum(pads, 1) - 1
        _, cache = w(inputs_embeds=[embs, None], position_ids=pos, q_blk=blk, q_valid=valid,
                     fill_cache_len=embs.shape[1])
        next_pos = pads.sum(-1)
        eos = getattr(self.language_tokenizer, "eos_token_id", 1) or 1
        mi_t, _ = self._indicator("Updated Memory: ", B, device, cfg.memory_indicator_max_length)
        memory, cache, next_pos = self._decode(cache, next_pos, mi_t, cfg.memory_max_length, eos)
        si_t, _ = self._indicator("Subtask: ", B, device, cfg.subtask_indicator_max_length)
        subtask, cache, next_pos = self._decode(cache, next_pos, si_t, cfg.response_max_length, eos)
        return memory, subtask


class PI07HighLevelPlannerPolicy(PreTrainedPolicy):
    config_class = PI07HighLevelPlannerConfig
    name = "pi07_high_level"
    model_class = PI07HighLevelPlannerModel

    @staticmethod
    def _vocab_size(config) -> int:
        vc = dict(config.vlm_config or {})
        return gemma3_4b_config(**{**vc.get("text", {}), **(config.vlm or {})}).vocab_size

    def __init__(self, config: PI07HighLevelPlannerConfig, per_dataset_stats=None, dataset_names=None, **_):
        super().__init__(config)
        n_heads = (len(per_dataset_stats) if per_dataset_stats is not None
                   else len(config.dataset_names) if config.dataset_names else 1)
        self.normalize_inputs = Normalize(config.input_features, config.normalization_mapping,
                                          per_dataset_stats=per_dataset_stats,
                                          dataset_names=dataset_names or config.dataset_names,
                                          num_datasets=None if per_dataset_stats is not None else n_heads,
                                          zero_range_center=config.zero_range_centers_on_zero,
                                          eps=config.normalization_epsilon)
        self.language_tokenizer = load_text_tokenizer(config.tokenizer_path, self._vocab_size(config))
        self.model = self.model_class(config, self.language_tokenizer)

    def reset(self) -> None:
        pass

    def get_optim_params(self):
        return [p for p in self.parameters() if p.requires_grad]

    def _tok(self, texts, max_len, device, key_tokens=None, batch=None):
        if batch is not None and key_tokens and f"{key_tokens}_tokens" in batch:
            return batch[f"{key_tokens}_tokens"].to(device), batch[f"{key_tokens}_masks"].to(device).bool()
        enc = self.language_tokenizer(list(texts), padding="max_length", padding_side="right", max_length=max_len,
                                      return_tensors="pt", truncation=True, add_special_tokens=False)
        return enc["input_ids"].to(device), enc["attention_mask"].to(device).bool()

    def _images(self, batch):
        cfg = self.config
        keys = [k for k in cfg.image_features] or sorted(k for k in batch if k.startswith("camera"))
        images, masks = [], []
        for i, k in enumerate(k for k in keys if k in batch):
            img = batch[k]
            img = img[:, -1] if img.dim() == 5 else img
            if tuple(img.shape[-2:]) != tuple(cfg.resize_imgs_with_padding):
                img = ops.resize_with_pad(img.float(), cfg.resize_imgs_with_padding[1], cfg.resize_imgs_with_padding[0], 0.0)
            images.append(img * 2.0 - 1.0)
            pad = batch.get("img_is_pad")
            masks.append(~pad[:, i].bool() if pad is not None else torch.ones(img.shape[0], dtype=torch.bool,
                                                                             device=img.device))
        return images, masks

    def _lang(self, batch, device):
        if "lang_tokens" in batch:
            return batch["lang_tokens"].to(device), batch["lang_masks"].to(device).bool()
        tasks = batch["prompt"]
        tasks = [tasks] if isinstance(tasks, str) else list(tasks)
        # "Task: ..., Past Memory: ..., State: <bins>, " (reference pi07/high_level_planner/modeling_pi07_high_level.py:
        # 749-760); the memory comes as ``past_memory`` (``memory`` is accepted too), the state part only with a state
        mems = batch.get("past_memory", batch.get("memory", [""] * len(tasks)))
        if "state" in batch:
            from ...pi05.modeling_pi05 import PI05Policy
            st = batch["state"].to(device)
            idx = self._resolve_dataset_index(batch, st.shape[0], device)
            normed = self.normalize_inputs({"state": st}, idx)            # the bins are cut on the NORMALISED state
            states = PI05Policy.prepare_discrete_state(self, normed)
            texts = [f"Task: {t}, Past Memory: {m}, State: {s}, " for t, m, s in zip(tasks, mems, states)]
        else:
            texts = [f"Task: {t}, Past Memory: {m}, " for t, m in zip(tasks, mems)]
        enc = self.language_tokenizer(texts, padding="max_length", padding_side="right",
                                      max_length=self.config.prompt_max_length, return_tensors="pt", truncation=True)
        return enc["input_ids"].to(device), enc["attention_mask"].to(device).bool()

    def forward(self, batch: dict[str, Any], return_per_sample: bool = False):
        device = next(self.parameters()).device
        images, masks = self._images(batch)
        lt, lm = self._lang(batch, device)
        B = lt.shape[0]
        cfg = self.config
        # targets close with the separator, so that decoding knows where a text ends
        mem_t, mem_m = self._tok([f"{m}<eos>" for m in batch.get("next_memory", [""] * B)], cfg.memory_max_length,
                                 device, "memory", batch)
        res_t, res_m = self._tok([f"{r}<eos>" for r in batch.get("response", [""] * B)], cfg.response_max_length,
                                 device, "response", batch)
        return self.model(images, masks, lt, lm, mem_t, mem_m, res_t, res_m, return_per_sample=return_per_sample)

    @torch.no_grad()
    def plan(self, batch: dict[str, Any]) -> tuple[list[str], list[str]]:
        """Returns ``(updated memory, subtask)`` strings per sample."""
        self.eval()
        device = next(self.parameters()).device
        images, masks = self._images(batch)
        lt, lm = self._lang(batch, device)
        mem, sub = self.model.generate(images, masks, lt, lm)
        dec = self.language_tokenizer.decode
        return [dec(r.tolist(), skip_special_tokens=True) for r in mem], \
               [dec(r.tolist(), skip_special_tokens=True) for r in sub]

    def select_action(self, batch):
        raise NotImplementedError("the high-level planner produces text (use .plan); actions come from pi07_low_level")
