"""Tensor-parallel prefix pass of the frozen Qwen3-VL backbone of cosmos3.

The reference runs the backbone as a black-box HF forward on every rank (``src/opentau/policies/cosmos3/
qwen3vl_with_expert.py:552-610``); at 32 B parameters that replicates 64 GB of frozen weights per GPU.  Here each
rank keeps 1/W of every backbone layer (:class:`~opentau_b200.parallel.tp.TPDecoderLayer`) and the ranks cooperate
on the union of their batches:

1. every rank embeds ITS OWN samples (vision tower and token embedding stay data parallel);
2. the decoder runs sequence-parallel over all ``B = W * B_local`` samples — a rank's row shard is exactly its own
   samples' tokens — with the all-gather and reduce-scatter fused into the qkv / gate-up and o / down GEMMs;
3. each layer leaves this rank's KV heads for ALL samples; one all-to-all at the end turns that into ALL heads for
   the rank's OWN samples, which is what the (data-parallel, trainable) action expert attends to.

Only layers the expert reads are exchanged (all of them, or the single ``condition_on_layer``).
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor

from ... import ops
from ...models.dual_stream import KVCache
from ...parallel.tp import TensorParallel, TPDecoderLayer


def _all_gather_cat(t: Tensor, tp: TensorParallel, dim: int = 0) -> Tensor:
    if tp.world == 1:
        return t
    parts = [torch.empty_like(t) for _ in range(tp.world)]
    dist.all_gather(parts, t.contiguous(), group=tp.group)
    return torch.cat(parts, dim)


class TPBackbone:
    """Sharded view of ``Qwen3VLWithExpertModel.backbone``'s decoder layers, built once."""

    def __init__(self, model, tp: TensorParallel, free_replicated_weights: bool = False):
        self.model, self.tp = model, tp
        lm = model.backbone.language_model
        self.layers = [TPDecoderLayer(layer, tp) for layer in lm.layers]
        if free_replicated_weights:
            for layer in lm.layers:                     # the sharded copies above are all that is needed from now on
                for lin in (layer.self_attn.qkv_proj, layer.self_attn.o_proj, layer.mlp.gate_up_proj, layer.mlp.down_proj):
                    lin.weight.data = lin.weight.data.new_empty(0)

    @torch.no_grad()
    def run_prefix(self, images, img_masks, lang_tokens, lang_masks) -> tuple[KVCache, Tensor]:
        m, tp = self.model, self.tp
        W, r = tp.world, tp.rank
        cfg = m.text_cfg
        embs, pad, pos, deep, n_img = m.backbone.embed_prefix(images, img_masks, lang_tokens, lang_masks)
        Bl, S, d = embs.shape
        B = Bl * W
        pad_all = _all_gather_cat(pad.to(torch.uint8), tp).bool()                  # (B, S)
        pos_all = _all_gather_cat(pos.permute(1, 0, 2).contiguous(), tp).permute(1, 0, 2).contiguous()   # (3, B, S)
        att = torch.ones(B, S, dtype=torch.bool, device=pad.device)
        blk, valid = ops.make_block_ids(pad_all, att)
        cos_sin = ops.mrope_angles(pos_all, cfg.head_dim, cfg.rope_theta, True, cfg.mrope_sections)
        col = m.condition_on_layer
        want = [col] if col is not None else list(range(len(self.layers)))
        x = embs.reshape(Bl * S, d)
        ks, vs = [], []
        for li, layer in enumerate(self.layers):
            x, k, v = layer(x, B, S, cos_sin, blk, valid)
            if deep is not None and li < len(deep):
                x = x.view(Bl, S, d)
                x = torch.cat([x[:, :n_img] + deep[li], x[:, n_img:]], dim=1).reshape(Bl * S, d)
            if li in want:
                ks.append(k), vs.append(v)
        k_all, v_all = torch.stack(ks), torch.stack(vs)                            # (L', B, S, hk_local, D)
        k_own, v_own = self._heads_for_own_samples(k_all, Bl), self._heads_for_own_samples(v_all, Bl)
        L_total = len(self.layers)
        # spare token slots behind the prefix, as the unsharded pass leaves them: the expert appends its keys / values
        # in place instead of concatenating in every layer of every denoise step
        room = 0 if torch.is_grad_enabled() else m.config.chunk_size + 8
        if col is not None or room:                                                # cache indexed by backbone layer id
            _, Bo, So, Ho, Do = k_own.shape
            k_full = k_own.new_zeros(L_total, Bo, So + room, Ho, Do)
            v_full = v_own.new_zeros(L_total, Bo, So + room, Ho, Do)
            if col is not None:
                k_full[col, :, :So], v_full[col, :, :So] = k_own[0], v_own[0]
            else:
                k_full[:, :, :So], v_full[:, :, :So] = k_own, v_own
            k_own, v_own = k_full, v_full
        return KVCache(k_own, v_own, pad, S), pos

    def _heads_for_own_samples(self, t: Tensor, Bl: int) -> Tensor:
        """``(L, B, S, hk_local, D)`` (my heads, all samples) -> ``(L, B_local, S, Hkv, D)`` (all heads, my samples)."""
        tp = self.tp
        W = tp.world
        if W == 1:
            return t
        L, B, S, hk, D = t.shape
        send = t.view(L, W, Bl, S, hk, D).permute(1, 0, 2, 3, 4, 5).contiguous()   # chunk w = samples of rank w
        recv = torch.empty_like(send)                                              # chunk w = heads of rank w, my samples
        dist.all_to_all_single(recv, send, group=tp.group) if t.is_cuda else self._all_to_all_gloo(recv, send)
        out = recv.permute(1, 2, 3, 0, 4, 5).reshape(L, Bl, S, W * hk, D)
        rep = self.layers[0].kv_rep
        if rep > 1:                                                                # KV heads were replicated over ranks
            out = out.view(L, Bl, S, W // rep, rep, hk, D)[:, :, :, :, 0].reshape(L, Bl, S, (W // rep) * hk, D)
        return out

    def _all_to_all_gloo(self, recv: Tensor, send: Tensor) -> None:
        """gloo has no all-to-all: gather everything and keep this rank's column."""
        tp = self.tp
        parts = [torch.empty_like(send) for _ in range(tp.world)]
        dist.all_gather(parts, send, group=tp.group)
        for w in range(tp.world):
            recv[w] = parts[w][tp.rank]
