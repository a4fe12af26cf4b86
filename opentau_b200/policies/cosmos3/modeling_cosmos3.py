"""cosmos3: frozen Qwen3-VL backbone supplying per-layer K/V to a trainable Qwen3 flow-matching expert.

Behaviour follows OpenTau ``src/opentau/policies/cosmos3/{qwen3vl_with_expert,modeling_cosmos3}.py``:
the backbone runs once under ``no_grad`` (causal over images + prompt) and its post-RoPE K/V are cached;
the expert (AdaRMS without a learned scale, per-head q/k norm, SwiGLU, interleaved MRoPE) sees
``[state token | 50 action tokens]``, attends to every valid prefix token and to its own block; suffix
positions continue after the largest prefix position on all three axes; the state token is conditioned
on time 1.0, action tokens on the flow time.  ``condition_on_layer = k`` truncates the backbone to k+1
layers and lets every expert layer read layer k's K/V (so the expert depth is free).  CE is zero.
State-dict keys: ``model.qwen3vl_with_expert.{backbone.*, expert.layers.N.*, expert.norm.*}``.
"""

from __future__ import annotations

from collections import deque
from typing import Any

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from ... import ops
from ...models.dual_stream import DualStreamDecoder, KVCache
from ...models.layers import Linear, Tower, TowerConfig
from ...models.qwen3vl import Qwen3VLBackbone, Qwen3VLVisionConfig, qwen3_text_config
from ...utils.tokenizer import load_text_tokenizer
from ..normalize import Normalize, Unnormalize
from ..pretrained import PreTrainedPolicy
from .configuration_cosmos3 import Cosmos3Config


class Qwen3VLWithExpertModel(nn.Module):
    def __init__(self, config: Cosmos3Config):
        super().__init__()
        self.config = config
        text = qwen3_text_config(**(config.backbone or {}))
        depth = text.num_hidden_layers
        col = config.condition_on_layer
        if col is not None:
            col = col % depth if col < 0 else col
            if not 0 <= col < depth:
                raise ValueError(f"condition_on_layer={config.condition_on_layer} outside the backbone depth {depth}")
            text.num_hidden_layers = col + 1          # deeper backbone layers are never needed
        elif config.expert_num_hidden_layers != depth:
            raise ValueError(f"expert depth ({config.expert_num_hidden_layers}) must equal the backbone depth "
                             f"({depth}) unless condition_on_layer is set")
        if config.expert_head_dim != text.head_dim or config.expert_num_key_value_heads != text.num_key_value_heads:
            raise ValueError("expert head_dim and num_key_value_heads must match the backbone's")
        self.condition_on_layer = col
        vis_over = dict(config.vision or {})
        vis_over.setdefault("out_hidden_size", text.hidden_size)
        vision = Qwen3VLVisionConfig(**vis_over)
        expert = TowerConfig(hidden_size=config.expert_hidden_size, num_hidden_layers=config.expert_num_hidden_layers,
                             num_attention_heads=config.expert_num_attention_heads,
                             num_key_value_heads=config.expert_num_key_value_heads, head_dim=config.expert_head_dim,
                             intermediate_size=config.expert_intermediate_size, vocab_size=text.vocab_size,
                             hidden_act="silu", rms_norm_eps=config.expert_rms_norm_eps,
                             rope_theta=text.rope_theta, norm_unit_offset=False, use_adarms=True,
                             adarms_cond_dim=config.expert_adarms_cond_dim, qk_norm=True, embed_scale=False,
                             mrope_sections=text.mrope_sections)
        self.text_cfg, self.expert_cfg, self.vision_cfg = text, expert, vision
        self.backbone = Qwen3VLBackbone(text, vision)
        self.expert = Tower(expert, with_embed=False)
        self.backbone_decoder = DualStreamDecoder([self.backbone.language_model], dropout=0.0)
        self.expert_decoder = DualStreamDecoder([self.expert], dropout=config.dropout,
                                                gradient_checkpointing=config.gradient_checkpointing)
        self.set_requires_grad()

    def set_requires_grad(self) -> None:
        c = self.config
        if c.train_expert_only:
            for p in self.backbone.parameters():
                p.requires_grad = False
        elif c.freeze_vision_encoder:
            for p in self.backbone.model.visual.parameters():
                p.requires_grad = False
        if c.train_vision_encoder_only:
            for p in self.parameters():
                p.requires_grad = False
            for p in self.backbone.model.visual.parameters():
                p.requires_grad = True
        if getattr(c, "train_state_action_representation_only", False):
            # no discrete-action pathway here: the whole wrapper is frozen, only the policy-level state / action
            # projections keep training
            from ..utils import freeze_with_expert_params_for_state_action_representation_only
            freeze_with_expert_params_for_state_action_representation_only(self)

    def train(self, mode: bool = True):
        super().train(mode)
        if self.config.train_expert_only:
            self.backbone.eval()
        return self

    def enable_tensor_parallel(self, tp, free_replicated_weights: bool = False) -> None:
        """Shards the (frozen) backbone decoder over the ranks of ``tp``; the prefix pass then runs tensor parallel
        over the union of the ranks' batches and returns each rank the KV cache of its own samples."""
        if any(p.requires_grad for p in self.backbone.language_model.parameters()):
            raise ValueError("tensor parallelism covers the frozen backbone only (train_expert_only=True)")
        from .tensor_parallel import TPBackbone
        self.tp_backbone = TPBackbone(self, tp, free_replicated_weights)

    def run_prefix(self, images, img_masks, lang_tokens, lang_masks) -> tuple[KVCache, Tensor]:
        """Backbone pass -> ``(cache, prefix positions (3,B,S))``; gradients only if the backbone trains."""
        if getattr(self, "tp_backbone", None) is not None:
            return self.tp_backbone.run_prefix(images, img_masks, lang_tokens, lang_masks)
        frozen = not any(p.requires_grad for p in self.backbone.parameters())
        with torch.set_grad_enabled(torch.is_grad_enabled() and not frozen):
            embs, pad, pos, deep, n_img = self.backbone.embed_prefix(images, img_masks, lang_tokens, lang_masks)
            B, S = pad.shape
            att = torch.ones(B, S, dtype=torch.bool, device=pad.device)      # fully causal
            blk, valid = ops.make_block_ids(pad, att)

            def hook(li, xs):
                if deep is not None and li < len(deep):
                    x = xs[0]
                    x = torch.cat([x[:, :n_img] + deep[li], x[:, n_img:]], dim=1)
                    return [x]
                return xs

            _, cache = self.backbone_decoder([embs], pos, blk, valid, fill_cache_len=S, mrope=True,
                                             layer_hook=hook if deep else None,
                                             cache_room=0 if torch.is_grad_enabled() else self.config.chunk_size + 8)
        return cache, pos

    def run_expert(self, cache: KVCache, suffix_embs: Tensor, suffix_pos: Tensor, cond: Tensor) -> Tensor:
        B, T, _ = suffix_embs.shape
        dev = suffix_embs.device
        pad = torch.ones(B, T, dtype=torch.bool, device=dev)
        att = torch.zeros(B, T, dtype=torch.bool, device=dev)
        att[:, 0] = True
        blk, valid = ops.make_block_ids(pad, att)
        layer_map = None
        if self.condition_on_layer is not None:
            layer_map = [self.condition_on_layer] * self.expert_cfg.num_hidden_layers
        (out,), _ = self.expert_decoder([suffix_embs], suffix_pos, blk, valid, adarms_cond=[cond], past=cache,
                                        mrope=True, past_layer_map=layer_map)
        return out


class Cosmos3FlowMatching(nn.Module):
    def __init__(self, config: Cosmos3Config):
        super().__init__()
        self.config = config
        self.qwen3vl_with_expert = Qwen3VLWithExpertModel(config)
        h, w = config.expert_hidden_size, config.proj_width
        self.action_in_proj = Linear(config.max_action_dim, h, bias=True)
        self.action_out_proj = Linear(h, config.max_action_dim, bias=True)
        self.time_mlp_in = Linear(w, w, bias=True)
        self.time_mlp_out = Linear(w, w, bias=True)
        self.adarms_proj = Linear(w, config.expert_adarms_cond_dim, bias=True)
        self.state_proj = Linear(config.max_state_dim, h, bias=True)

    @staticmethod
    def sample_noise(shape, device) -> Tensor:
        return torch.randn(shape, dtype=torch.float32, device=device)

    @staticmethod
    def sample_time(bsize: int, device) -> Tensor:
        u = torch.rand(bsize, dtype=torch.float32, device=device).clamp_min(1e-12)
        return u.pow(1.0 / 1.5) * 0.999 + 0.001

    def _time_to_adarms(self, time: Tensor) -> Tensor:
        """``(B, N)`` times -> ``(B, N, cond_dim)`` conditioning vectors."""
        dtype = self.action_in_proj.weight.dtype
        e = ops.sinusoidal_time_embedding(time, self.config.proj_width, 4e-3, 4.0, out_dtype=dtype)
        x = F.silu(self.time_mlp_in(e))
        x = F.silu(self.time_mlp_out(x))
        return self.adarms_proj(x)

    def embed_suffix(self, noisy_actions: Tensor, timestep: Tensor, state: Tensor):
        dtype = self.action_in_proj.weight.dtype
        B = noisy_actions.shape[0]
        a = self.action_in_proj(noisy_actions.to(dtype))
        s = self.state_proj(state.to(dtype))[:, None, :]
        embs = torch.cat([s, a], dim=1)
        t_full = torch.cat([torch.ones(B, 1, dtype=torch.float32, device=a.device), timestep.float()], dim=1)
        return embs, self._time_to_adarms(t_full)

    @staticmethod
    def _suffix_positions(prefix_pos: Tensor, n: int) -> Tensor:
        off = prefix_pos.amax(dim=(0, 2)) + 1
        suf = off[:, None] + torch.arange(n, device=prefix_pos.device)[None, :]
        return suf[None].expand(3, -1, -1)

    def _run_expert(self, cache, prefix_pos, x_t, time, state) -> Tensor:
        embs, cond = self.embed_suffix(x_t, time, state)
        pos = self._suffix_positions(prefix_pos, embs.shape[1])
        out = self.qwen3vl_with_expert.run_expert(cache, embs, pos, cond)
        return self.action_out_proj(out[:, -self.config.chunk_size:]).float()

    def forward(self, images, img_masks, lang_tokens, lang_masks, state, actions, actions_is_pad=None, noise=None,
                time=None, real_action_dim=None, return_per_sample=False):
        cfg = self.config
        B, device = actions.shape[0], actions.device
        cache, ppos = self.qwen3vl_with_expert.run_prefix(images, img_masks, lang_tokens, lang_masks)
        cache = cache.detach()
        actions = actions.float()
        noise = self.sample_noise(actions.shape, device) if noise is None else noise.float()
        time = self.sample_time(B, device) if time is None else time
        if cfg.max_delay > 0:
            delay = torch.randint(0, cfg.max_delay + 1, (B,), device=device)
            frozen = torch.arange(cfg.chunk_size, device=device)[None, :] < delay[:, None]
        else:
            frozen = torch.zeros(B, cfg.chunk_size, dtype=torch.bool, device=device)
        t2 = torch.where(frozen, torch.zeros((), device=device), time[:, None])
        x_t, u_t = ops.flow_interpolate(actions, noise, t2)
        v_t = self._run_expert(cache, ppos, x_t, t2, state)
        mse = ops.flow_matching_masked_mse(u_t, v_t, frozen, actions_is_pad, real_action_dim, return_per_sample)
        loss, per = mse if return_per_sample else (mse, None)
        out = {"MSE": loss, "CE": torch.zeros((), device=device, dtype=loss.dtype)}
        if return_per_sample:
            z = torch.zeros(B, device=device)
            out["MSE_per_sample"], out["CE_per_sample"] = per, (z, z.clone())
        return out

    def executed_rows(self, batch: int, device, frozen: Tensor | None = None) -> Tensor:
        """``(B, chunk)`` bool rows that are executed: not frozen and inside the first ``n_action_steps`` live rows."""
        from ..accel import executed_row_mask
        cfg = self.config
        if frozen is None:
            frozen = torch.zeros(batch, cfg.chunk_size, dtype=torch.bool, device=device)
        return executed_row_mask(prefix_mask=frozen, delay=frozen.sum(dim=1), chunk_size=cfg.chunk_size,
                                 n_action_steps=cfg.n_action_steps, device=device)

    @torch.no_grad()
    def sample_actions(self, images, img_masks, lang_tokens, lang_masks, state, noise=None, action_prefix=None,
                       frozen=None, n_candidates: int = 1, accel=None) -> Tensor:
        cfg = self.config
        B, device = lang_tokens.shape[0], lang_tokens.device
        if noise is None:
            noise = self.sample_noise((B * n_candidates, cfg.chunk_size, cfg.max_action_dim), device)
        cache, ppos = self.qwen3vl_with_expert.run_prefix(images, img_masks, lang_tokens, lang_masks)
        if n_candidates > 1:
            cache = cache.expand_batch(n_candidates)
            ppos = ppos.repeat_interleave(n_candidates, 1)
            state = state.repeat_interleave(n_candidates, 0)
        return self.denoise_loop(cache, ppos, state, noise, action_prefix, frozen, accel)

    @torch.no_grad()
    def denoise_loop(self, cache, ppos, state, noise, action_prefix=None, frozen=None, accel=None) -> Tensor:
        """``num_steps`` Euler steps of the expert over a finished prefix cache: fixed trip count, device-only
        operations and no collective, so the loop can be replayed from a CUDA graph also when the backbone that
        produced the cache runs tensor parallel."""
        cfg = self.config
        device = noise.device
        x_t = noise.float().clone()
        Bn = x_t.shape[0]
        if frozen is None:
            frozen = torch.zeros(Bn, cfg.chunk_size, dtype=torch.bool, device=device)
        live = (~frozen).float()
        if accel is not None:
            accel.set_row_mask(self.executed_rows(Bn, device, frozen))
        dt = -1.0 / cfg.num_steps
        if action_prefix is not None:
            x_t = torch.where(frozen[:, :, None], action_prefix.float(), x_t)
        for i in range(cfg.num_steps):
            v_t = self._run_expert(cache, ppos, x_t, live * (1.0 + i * dt), state)
            if accel is not None:
                accel.update(v_t)
            x_t = ops.euler_step(x_t, v_t, dt, frozen if action_prefix is not None else None, action_prefix)
        return x_t


class Cosmos3Policy(PreTrainedPolicy):
    config_class = Cosmos3Config
    name = "cosmos3"

    def __init__(self, config: Cosmos3Config, per_dataset_stats: list[dict] | None = None,
                 dataset_names: list[str] | None = None, **_):
        super().__init__(config)
        n_heads = (len(per_dataset_stats) if per_dataset_stats is not None
                   else len(config.dataset_names) if config.dataset_names else 1)
        kw = dict(per_dataset_stats=per_dataset_stats, dataset_names=dataset_names or config.dataset_names,
                  num_datasets=None if per_dataset_stats is not None else n_heads,
                  zero_range_center=config.zero_range_centers_on_zero, eps=config.normalization_epsilon)
        self.normalize_inputs = Normalize(config.input_features, config.normalization_mapping, **kw)
        self.normalize_targets = Normalize(config.output_features, config.normalization_mapping, **kw)
        self.unnormalize_outputs = Unnormalize(config.output_features, config.normalization_mapping, **kw)
        vocab = qwen3_text_config(**(config.backbone or {})).vocab_size
        self.language_tokenizer = load_text_tokenizer(config.tokenizer_path, vocab)
        self.model = Cosmos3FlowMatching(config)
        from ..utils import apply_policy_level_freezes
        apply_policy_level_freezes(self.model, self.model.qwen3vl_with_expert, config)
        self.accel_prefix: int | None = None       # armed by accel.configure_accel
        self.last_accel_provenance = None
        self.last_candidate_scores = None
        self._n_candidates, self._critic = 1, None  # armed by candidates.configure_candidates
        self.reset()

    def enable_tensor_parallel(self, tp, free_replicated_weights: bool = False) -> None:
        self.model.qwen3vl_with_expert.enable_tensor_parallel(tp, free_replicated_weights)

    def reset(self) -> None:
        self._action_queue: deque = deque([], maxlen=self.config.n_action_steps)
        self.last_accel = None
        self.last_accel_candidates = None

    def get_optim_params(self):
        return [p for p in self.parameters() if p.requires_grad]

    def prepare_images(self, batch) -> tuple[list[Tensor], list[Tensor]]:
        size = self.config.image_resize
        keys = [k for k in self.config.image_features] or sorted(k for k in batch if k.startswith("camera"))
        images, masks = [], []
        pad_flags = batch.get("img_is_pad")
        for i, k in enumerate(k for k in keys if k in batch):
            img = batch[k]
            img = img[:, -1] if img.dim() == 5 else img
            if tuple(img.shape[-2:]) != (size, size):
                img = ops.resize_with_pad(img.float(), size, size, pad_value=0.0)
            images.append(img * 2.0 - 1.0)
            B = img.shape[0]
            masks.append(~pad_flags[:, i].bool() if pad_flags is not None
                         else torch.ones(B, dtype=torch.bool, device=img.device))
        if not images:
            raise ValueError("no camera images in the batch")
        return images, masks

    def prepare_language(self, batch) -> tuple[Tensor, Tensor]:
        device = batch["state"].device
        if "lang_tokens" in batch:
            return batch["lang_tokens"].to(device), batch["lang_masks"].to(device).bool()
        tasks = batch["prompt"]
        tasks = [tasks] if isinstance(tasks, str) else list(tasks)
        enc = self.language_tokenizer(tasks, padding="max_length", padding_side="right",
                                      max_length=self.config.prompt_max_length, return_tensors="pt", truncation=True)
        return enc["input_ids"].to(device), enc["attention_mask"].to(device).bool()

    def _common(self, batch):
        B, device = batch["state"].shape[0], batch["state"].device
        idx = self._resolve_dataset_index(batch, B, device)
        nb = self.normalize_inputs(batch, idx)
        images, masks = self.prepare_images(nb)
        lt, lm = self.prepare_language(nb)
        state = nb["state"][:, -1] if nb["state"].dim() == 3 else nb["state"]
        return idx, images, masks, lt, lm, state

    def forward(self, batch, noise=None, time=None, return_per_sample: bool = False):
        idx, images, masks, lt, lm, state = self._common(batch)
        tb = self.normalize_targets(batch, idx)
        return self.model(images, masks, lt, lm, state, tb["actions"], actions_is_pad=batch.get("action_is_pad"),
                          noise=noise, time=time, real_action_dim=batch.get("real_action_dim"),
                          return_per_sample=return_per_sample)

    @torch.no_grad()
    def sample_actions(self, batch, noise=None, n_candidates: int | None = None, **_) -> Tensor:
        """Un-normalised action chunk ``(B, chunk, real_dim)``; best-of-N and the accel score as in the pi0.5 wrapper
        (reference ``src/opentau/policies/cosmos3/modeling_cosmos3.py`` ``sample_actions``)."""
        from ..accel import make_meter, publish
        from ..candidates import (MEDOID, MedoidCritic, expand_candidates, pick, select_candidate,
                                  warn_if_no_candidate_scored)
        self.eval()
        cfg = self.config
        idx, images, masks, lt, lm, state = self._common(batch)
        B, device = lt.shape[0], lt.device
        n = int(n_candidates or getattr(self, "_n_candidates", None) or 1)
        critic = getattr(self, "_critic", None)
        if n > 1 and critic is None:
            if getattr(cfg, "action_chunk_critic_path", None) not in (None, MEDOID):
                raise ValueError(f"n_candidates={n} but no action-chunk critic is attached; arm best-of-N through "
                                 "candidates.configure_candidates")
            critic = MedoidCritic(self.unnormalize_outputs, max_action_dim=cfg.max_action_dim)
        sampler_idx = expand_candidates(idx, n)
        meter = make_meter(self, batch_size=B * n, device=device, dataset_index=sampler_idx)
        if getattr(self, "_use_graphs", False) and device.type == "cuda" and meter is None and n == 1:
            actions = self._graphed_sample(images, masks, lt, lm, state, noise)
        else:
            actions = self.model.sample_actions(images, masks, lt, lm, state, noise=noise, n_candidates=n, accel=meter)
        if n == 1:
            publish(self, meter, dataset_index=idx)
        feat = cfg.action_feature
        real = feat.shape[0] if feat is not None else actions.shape[-1]
        actions = self.unnormalize_outputs({"actions": actions[:, :, :real]}, sampler_idx)["actions"]
        if n == 1:
            return actions
        candidates = actions.view(B, n, *actions.shape[1:])
        scores = critic.score_chunks(batch, candidates, row_mask=self.model.executed_rows(B, device),
                                     dataset_index=idx)
        selected = select_candidate(scores)
        self.last_candidate_scores = scores.detach().to(torch.float32).cpu().tolist()
        warn_if_no_candidate_scored(self.last_candidate_scores)
        publish(self, meter, dataset_index=sampler_idx, n_candidates=n, selected=selected)
        return pick(candidates, selected)

    def enable_cuda_graphs(self, flag: bool = True) -> None:
        """Replay the sampler (backbone prefix pass + Euler loop over the expert) from one CUDA graph per input
        signature; the reference's counterpart is ``torch.compile(mode="reduce-overhead")``
        (``src/opentau/scripts/benchmark_inference.py:249-259``)."""
        self._use_graphs = bool(flag)
        self._graph_runner = None
        self._loop_runner = None

    def _graphed_sample(self, images, masks, lt, lm, state, noise):
        from ...models.dual_stream import KVCache
        from ...runtime.graphs import CudaGraphRunner
        cfg = self.config
        if noise is None:
            noise = self.model.sample_noise((lt.shape[0], cfg.chunk_size, cfg.max_action_dim), lt.device)
        if getattr(self.model.qwen3vl_with_expert, "tp_backbone", None) is not None:
            # tensor-parallel backbone: its kernels carry a per-call epoch in their arguments and its pass contains
            # library collectives, so the prefix pass runs eagerly; the expert loop behind it touches no peer and
            # is replayed from a graph whose inputs are the cache tensors
            cache, ppos = self.model.qwen3vl_with_expert.run_prefix(images, masks, lt, lm)
            length = cache.length
            if getattr(self, "_loop_runner", None) is None:
                def loop(k, v, valid, ppos, state, noise):
                    return self.model.denoise_loop(KVCache(k, v, valid, length), ppos, state, noise)
                self._loop_runner, self._loop_length = CudaGraphRunner(loop), length
            if length != self._loop_length:
                raise RuntimeError(f"prefix length changed from {self._loop_length} to {length}: the captured expert "
                                   "loop is for one prompt / camera geometry; call enable_cuda_graphs(True) again")
            return self._loop_runner(cache.k, cache.v, cache.valid, ppos, state, noise.float()).clone()
        if getattr(self, "_graph_runner", None) is None:
            def fn(images, masks, lt, lm, state, noise):
                return self.model.sample_actions(list(images), list(masks), lt, lm, state, noise=noise)
            self._graph_runner = CudaGraphRunner(fn)
        return self._graph_runner(tuple(images), tuple(masks), lt, lm.bool(), state, noise.float()).clone()

    @torch.no_grad()
    def select_action(self, batch, noise=None) -> Tensor:
        if len(self._action_queue) == 0:
            actions = self.sample_actions(batch, noise=noise)
            self._action_queue.extend(actions.transpose(0, 1)[: self.config.n_action_steps])
        return self._action_queue.popleft()
