"""pi0: PaliGemma backbone and a Gemma-300M action expert trained jointly (no knowledge insulation).

Suffix = ``[state token, 50 action tokens]`` where each action token is ``MLP([action_in_proj(x_t) || time_emb])``;
the expert uses plain RMSNorm (time enters through the tokens, not through adaptive norms).  Training runs
ONE pass over ``[prefix | suffix]`` with the block mask ``prefix (bidirectional) < state < actions``;
inference caches the prefix K/V and runs the expert alone.  The loss is the masked flow-matching MSE,
optionally weighted by ``min(exp(advantage), awr_max_weight)``; ``CE`` is identically zero
(reference ``src/opentau/policies/pi0/modeling_pi0.py:174-975``).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor

from ... import ops
from ...models.layers import Linear
from ..pi05.modeling_pi05 import (PI05FlowMatching, PI05Policy, PaliGemmaWithExpertModel, gemma_300m_config)
from .configuration_pi0 import PI0Config


class _PI0Wrapper(PaliGemmaWithExpertModel):
    def __init__(self, config):
        over = dict(config.expert or {})
        over.setdefault("use_adarms", False)
        config_expert_backup = config.expert
        config.expert = over
        try:
            super().__init__(config)
        finally:
            config.expert = config_expert_backup


class PI0FlowMatching(PI05FlowMatching):
    def build_wrapper(self, config):
        return _PI0Wrapper(config)

    def __init__(self, config: PI0Config, tokenizer=None):
        super().__init__(config, tokenizer)
        w = self.wrapper.expert_cfg.hidden_size
        # pi0 replaces the time MLP by an action||time MLP and always has a state projection (into the expert)
        del self.time_mlp_in, self.time_mlp_out
        if hasattr(self, "state_proj"):
            del self.state_proj
        self.state_proj = Linear(config.max_state_dim, w, bias=True)
        self.action_time_mlp_in = Linear(2 * w, w, bias=True)
        self.action_time_mlp_out = Linear(w, w, bias=True)

    def embed_prefix(self, images, img_masks, lang_tokens, lang_masks, *a, **kw):
        kw.pop("state", None)
        state_type = self.config.state_type
        self.config.state_type = "discrete"     # the pi0 prefix never holds a state token
        try:
            return super().embed_prefix(images, img_masks, lang_tokens, lang_masks, None, None, None, None, state=None)
        finally:
            self.config.state_type = state_type

    def embed_suffix(self, state: Tensor, noisy_actions: Tensor, timestep: Tensor):
        """``timestep (B,)`` or ``(B, T)``.  Returns ``(embs, pad, att)`` with att ``[1, 1, 0, ...]``."""
        dtype = self.action_in_proj.weight.dtype
        B, T = noisy_actions.shape[:2]
        device = noisy_actions.device
        w = self.action_in_proj.out_features
        state_emb = self.state_proj(state.to(dtype))[:, None, :]
        t2 = timestep if timestep.dim() == 2 else timestep[:, None].expand(B, T)
        time_emb = ops.sinusoidal_time_embedding(t2, w, 4e-3, 4.0, out_dtype=dtype)
        action_emb = self.action_in_proj(noisy_actions.to(dtype))
        h = self.action_time_mlp_out(F.silu(self.action_time_mlp_in(torch.cat([action_emb, time_emb], dim=2))))
        embs = torch.cat([state_emb, h], dim=1)
        pad = torch.ones(B, T + 1, dtype=torch.bool, device=device)
        att = torch.zeros(B, T + 1, dtype=torch.bool, device=device)
        att[:, :2] = True
        return embs, pad, att

    def forward(self, images, img_masks, lang_tokens, lang_masks, actions, actions_is_pad=None, noise=None,
                time=None, state=None, real_action_dim=None, advantage=None, return_per_sample=False, **_):
        cfg = self.config
        B = actions.shape[0]
        device = actions.device
        actions = actions.float()
        noise = self.sample_noise(actions.shape, device) if noise is None else noise.float()
        time = self.sample_time(B, device) if time is None else time
        t2 = time[:, None].expand(B, cfg.chunk_size)
        x_t, u_t = ops.flow_interpolate(actions, noise, t2)
        pe, pp, pa, _ = self.embed_prefix(images, img_masks, lang_tokens, lang_masks)
        se, sp, sa = self.embed_suffix(state, x_t, time)
        pad = torch.cat([pp, sp], 1)
        att = torch.cat([pa, sa], 1)
        blk, valid = ops.make_block_ids(pad, att)
        pos = torch.cumsum(pad, 1) - 1
        (_, so), _ = self.wrapper(inputs_embeds=[pe, se], position_ids=pos, q_blk=blk, q_valid=valid)
        v_t = self.action_out_proj(so[:, -cfg.chunk_size:]).float()
        mask = torch.ones_like(u_t, dtype=torch.bool)
        if actions_is_pad is not None:
            mask &= ~actions_is_pad.bool()[:, :, None]
        if real_action_dim is not None:
            mask &= torch.arange(u_t.shape[-1], device=device)[None, None, :] < real_action_dim.view(B, 1, 1)
        se2 = (u_t - v_t).pow(2) * mask
        if cfg.use_awr and advantage is not None:
            wgt = torch.clamp(torch.exp(advantage.float()), max=cfg.awr_max_weight)
            se2 = se2 * wgt.view(B, 1, 1)
        loss = se2.sum() / (mask.sum() + 1e-8)
        out = {"MSE": loss, "CE": torch.zeros_like(loss)}
        if return_per_sample:
            z = torch.zeros(B, device=device)
            out["MSE_per_sample"] = (se2.sum(dim=(1, 2)), mask.sum(dim=(1, 2)).float())
            out["CE_per_sample"] = (z, z.clone())
        return out

    @torch.no_grad()
    def denoise_step(self, cache, prefix_len, x_t, time, state=None):
        se, sp, sa = self.embed_suffix(self._state, x_t, time)
        s_blk, s_valid = ops.make_block_ids(sp, sa)
        s_pos = prefix_len + torch.cumsum(sp, dim=1) - 1
        (_, so), _ = self.wrapper(inputs_embeds=[None, se], position_ids=s_pos, q_blk=s_blk, q_valid=s_valid,
                                  past=cache)
        return self.action_out_proj(so[:, -self.config.chunk_size:]).float()

    @torch.no_grad()
    def sample_actions(self, images, img_masks, lang_tokens, lang_masks, action_prefix=None, delay=0, noise=None,
                       state=None, n_candidates: int = 1, accel=None, frozen=None, prefix_kwargs=None):
        if state is None:
            raise ValueError("pi0 needs the state vector at inference")
        self._state = state.repeat_interleave(n_candidates, 0) if n_candidates > 1 else state
        try:
            return super().sample_actions(images, img_masks, lang_tokens, lang_masks, action_prefix, delay, noise,
                                          None, n_candidates, accel, frozen, prefix_kwargs)
        finally:
            self._state = None


class PI0Policy(PI05Policy):
    config_class = PI0Config
    name = "pi0"
    model_class = PI0FlowMatching
    _TILE_LINEAR_INPUTS = True       # older checkpoints have narrower state / action inputs (reference pi0/modeling_pi0.py:354)

    def prepare_language(self, batch):
        cfg = self.config
        device = batch["state"].device
        if "lang_tokens" in batch:
            return batch["lang_tokens"].to(device), batch["lang_masks"].to(device).bool()
        tasks = batch["prompt"]
        tasks = [tasks] if isinstance(tasks, str) else list(tasks)
        tasks = [t if t.endswith("\n") else f"{t}\n" for t in tasks]
        for i, t in enumerate(tasks):
            if cfg.advantage == "on":
                tasks[i] = f"{t}Advantage: positive\n"
            elif cfg.advantage == "use":
                pos = True if "advantage" not in batch else bool(batch["advantage"][i] >= cfg.advantage_threshold)
                tasks[i] = f"{t}Advantage: {'positive' if pos else 'negative'}\n"
        enc = self.language_tokenizer(tasks, padding="max_length", padding_side="right",
                                      max_length=cfg.tokenizer_max_length, return_tensors="pt", truncation=True)
        return enc["input_ids"].to(device), enc["attention_mask"].to(device).bool()

    def forward(self, batch, noise=None, time=None, return_per_sample: bool = False):
        B = batch["state"].shape[0]
        device = batch["state"].device
        idx = self._resolve_dataset_index(batch, B, device)
        nb = self.normalize_inputs(batch, idx)
        tb = self.normalize_targets(batch, idx)
        images, img_masks = self.prepare_images(nb)
        lang_tokens, lang_masks = self.prepare_language(nb)
        state = nb["state"][:, -1] if nb["state"].dim() == 3 else nb["state"]
        return self.model(images, img_masks, lang_tokens, lang_masks, tb["actions"],
                          actions_is_pad=batch.get("action_is_pad"), noise=noise, time=time, state=state,
                          real_action_dim=batch.get("real_action_dim"), advantage=batch.get("advantage"),
                          return_per_sample=return_per_sample)
