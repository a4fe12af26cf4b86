"""Interleaved two-tower decoder: a VLM backbone and an action expert that share attention.

Each layer projects q/k/v per tower, concatenates the present towers along the token axis,
applies RoPE, optionally prepends cached (already rotated) prefix keys/values, runs ONE
block-causal attention and sends each tower's slice back through its own output projection
and MLP.  This covers the three reference wrappers with one implementation
(OpenTau ``policies/pi05/paligemma_with_expert.py:549-803``,
``policies/pi07/gemma3_with_expert.py:419-584``, ``policies/cosmos3/qwen3vl_with_expert.py:208-342``).

The KV cache is a pre-allocated ``(L, B, S_max, Hkv, D)`` pair per model instead of a
dict grown by concatenation, so the denoise loop has static shapes and can be graph captured.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import Tensor, nn

from .. import ops
from .layers import AdaRMSNorm, DecoderLayer, Tower, TowerConfig


@dataclass
class KVCache:
    """Post-RoPE keys/values of the first ``length`` prefix tokens for every layer."""

    k: Tensor  # (L, B, S, Hkv, D)
    v: Tensor
    valid: Tensor  # (B, S) bool: pad mask of the cached tokens
    length: int

    def detach(self) -> "KVCache":
        return KVCache(self.k.detach(), self.v.detach(), self.valid, self.length)

    def expand_batch(self, n: int) -> "KVCache":
        """Widen a batch-1 cache to ``n`` candidates that share the prefix (best-of-N)."""
        L, B, S, H, D = self.k.shape
        return KVCache(self.k.expand(L, n, S, H, D) if B == 1 else self.k.repeat_interleave(n, 1),
                       self.v.expand(L, n, S, H, D) if B == 1 else self.v.repeat_interleave(n, 1),
                       self.valid.expand(n, self.valid.shape[1]) if B == 1 else self.valid.repeat_interleave(n, 0),
                       self.length)

    def writable_room(self) -> int:
        """Tokens that fit behind the cached prefix in place (0 when the buffers are expanded views)."""
        k = self.k
        dense = k.stride(4) == 1 and k.stride(3) == k.shape[4] and k.stride(2) == k.shape[3] * k.shape[4] \
            and k.stride(1) >= k.shape[2] * k.stride(2)
        return k.shape[2] - self.length if dense and self.v.stride() == k.stride() else 0


class DualStreamDecoder(nn.Module):
    """Runs ``towers[i]`` over ``inputs_embeds[i]`` (``None`` = tower absent in this pass)."""

    def __init__(self, towers: list[Tower], dropout: float = 0.0, same_theta_for_all: bool = True,
                 gradient_checkpointing: bool = False):
        super().__init__()
        self.towers = towers  # plain list: the owning wrapper registers the modules under HF names
        self.dropout = nn.Dropout(dropout)
        self.gradient_checkpointing = gradient_checkpointing
        n = {t.cfg.num_hidden_layers for t in towers}
        if len(n) != 1:
            raise ValueError(f"towers must have the same depth, got {n}")
        self.num_layers = n.pop()
        # set by the parameter-sharded engine (parallel/fsdp.py): makes a layer's weights resident before the layer
        # runs and before its backward pass; None for replicated parameters
        self.param_gate = None

    # -- adaptive-norm conditions: one GEMM for all layers of a tower ------------------------------
    @staticmethod
    def _ada_mods(tower: Tower, cond: Tensor | None) -> list | None:
        """Pre-computes ``dense(cond)`` of every adaptive norm of ``tower`` in one GEMM.

        The condition is the same for every layer, so the 2L+1 small GEMMs collapse into one
        ``[rows, cond] x [cond, (2L+1)*3H]`` product.  Returns per-layer tuples of slices.
        """
        if cond is None or not tower.cfg.use_adarms:
            return None
        norms: list[AdaRMSNorm] = []
        for layer in tower.layers:
            norms += [layer.input_layernorm, layer.post_attention_layernorm]
        norms.append(tower.norm)
        w, b = DualStreamDecoder._stacked_dense(tower, norms)
        out = ops.linear(cond.to(w.dtype), w, b)
        chunks = out.split(3 * tower.cfg.hidden_size, dim=-1)
        return list(chunks)

    @staticmethod
    def _stacked_dense(tower: Tower, norms: list) -> tuple[Tensor, Tensor]:
        """Weights / biases of all adaptive-norm projections of a tower as ONE matrix and ONE vector.

        Training (or parameters owned by a flat training buffer): concatenated per call, so autograd and the optimizer
        see the individual parameters.  Inference: the parameters are re-homed ONCE as views of a stacked buffer (a
        deep tower's stack is hundreds of MB: concatenating it for every denoise step cost more than the product that
        consumes it).  In-place updates (``load_state_dict``) write through the views, so neither eager calls nor a
        captured CUDA graph can see stale values; a dtype / device move re-allocates the parameters, which the
        pointer check below notices."""
        ws, bs = [n.dense.weight for n in norms], [n.dense.bias for n in norms]
        managed = any(hasattr(p, "main_grad") for p in ws + bs)
        if managed or (torch.is_grad_enabled() and any(p.requires_grad for p in ws + bs)):
            return torch.cat(ws, dim=0), torch.cat(bs, dim=0)
        stack = getattr(tower, "_ada_stack", None)
        rows = [p.shape[0] for p in ws]

        def is_view(buf: Tensor, parts: list, row_elems: int) -> bool:
            off = 0
            for p in parts:
                if p.dtype != buf.dtype or p.device != buf.device or \
                        p.data_ptr() != buf.data_ptr() + off * row_elems * buf.element_size():
                    return False
                off += p.shape[0]
            return True

        if stack is None or not (is_view(stack[0], ws, ws[0].shape[1]) and is_view(stack[1], bs, 1)):
            with torch.no_grad():
                w_all, b_all = torch.cat(ws, dim=0), torch.cat(bs, dim=0)
                off = 0
                for p, pb, r in zip(ws, bs, rows):
                    p.data, pb.data = w_all[off:off + r], b_all[off:off + r]
                    off += r
            stack = (w_all, b_all)
            tower._ada_stack = stack
        return stack

    def _layer(self, li: int, xs: list[Tensor | None], cos_sin, q_blk, k_blk, q_valid, k_valid,
               cache_k, cache_v, mods, kv_dst=None, cp=None) -> tuple[list[Tensor | None], Tensor | None, Tensor | None]:
        """``kv_dst = (k_buf, v_buf, offset)``: inference with one tower present writes the new keys / values into
        these ``(B, S_buf, Hkv, D)`` buffers at ``offset`` (behind a cached prefix, or at 0 when a cache is being
        filled) and attends over ``[:offset + T]`` in place: no concatenation, no copy."""
        towers = self.towers
        xs = list(xs)                       # the forked norms below replace entries; the caller's list stays as it is
        qs, ks, vs, gates1, lens = [], [], [], [], []
        present = [(tower, x) for tower, x in zip(towers, xs) if x is not None]
        cos, sin = cos_sin
        fused_post = len(present) == 1 and ops.can_fuse_qkv_post(present[0][1], present[0][0].cfg.head_dim)
        for ti, (tower, x) in enumerate(zip(towers, xs)):
            if x is None:
                continue
            layer: DecoderLayer = tower.layers[li]
            # forked norms: the residual connection takes the norm's second output, so that the two gradients of the
            # residual stream are summed inside the norm's backward kernel
            fork = torch.is_grad_enabled()
            if mods[ti] is not None:
                h, g1, *xr = layer.input_layernorm(x, precomputed=mods[ti][2 * li], fork=fork)
            else:
                h, g1, *xr = layer.input_layernorm(x, fork=fork)
            if xr:
                xs[ti] = xr[0]
            gates1.append(g1), lens.append(x.shape[1])
            if fused_post:
                # one kernel: split + qk-norm + rotation + K/V store (into the cache when there is room)
                attn, cfg = layer.self_attn, tower.cfg
                T = x.shape[1]
                k_dst = v_dst = None
                if kv_dst is not None:
                    off = kv_dst[2]
                    k_dst, v_dst = kv_dst[0][:, off:off + T], kv_dst[1][:, off:off + T]
                q, new_k, new_v = ops.qkv_post(attn.qkv_proj(h), cfg.num_attention_heads, cfg.num_key_value_heads,
                                               cfg.head_dim, attn.q_norm if cfg.qk_norm else None,
                                               attn.k_norm if cfg.qk_norm else None, cos, sin, k_dst, v_dst)
                if kv_dst is not None:
                    k, v = kv_dst[0][:, :off + T], kv_dst[1][:, :off + T]
                elif cache_k is not None:
                    k, v = ops.seq_concat(cache_k, new_k), ops.seq_concat(cache_v, new_v)
                else:
                    k, v = new_k, new_v
                continue
            q, k, v = layer.self_attn.qkv(h)
            qs.append(q), ks.append(k), vs.append(v)
        if not fused_post:
            q = qs[0] if len(qs) == 1 else torch.cat(qs, dim=1)
            k = ks[0] if len(ks) == 1 else torch.cat(ks, dim=1)
            v = vs[0] if len(vs) == 1 else torch.cat(vs, dim=1)
            q = ops.rope(q, cos, sin)
            k = ops.rope(k, cos, sin)
            new_k, new_v = k, v
            if cache_k is not None:
                k = ops.seq_concat(cache_k, k)
                v = ops.seq_concat(cache_v, v)
        first = next(t for t, x in zip(towers, xs) if x is not None)
        if cp is not None:
            # the sequence is sharded over the ranks: q / k / v are this rank's slice, k_blk / k_valid cover all keys
            att = cp.attention(q, k, v, q_blk, k_blk, q_valid, k_valid, first.cfg.attn_scale)
        else:
            att = ops.block_attention(q, k, v, q_blk, k_blk, q_valid, k_valid, first.cfg.attn_scale)
        outs: list[Tensor | None] = []
        start, j = 0, 0
        for ti, (tower, x) in enumerate(zip(towers, xs)):
            if x is None:
                outs.append(None)
                continue
            layer = tower.layers[li]
            cfg = tower.cfg
            a = att[:, start:start + lens[j]]
            start += lens[j]
            g1 = gates1[j]
            j += 1
            drop = self.dropout if self.training and self.dropout.p > 0 else None
            if cfg.sandwich_norms:
                # Gemma-3: x + post_attn_norm(o_proj(att)); x + post_ffw_norm(mlp(pre_ffw_norm(x)))
                o = layer.self_attn.o_proj(a)
                if drop is not None:
                    o = drop(o)
                y = x + layer.post_attention_layernorm(o)[0]
                n, _, *yr = layer.pre_feedforward_layernorm(y, fork=torch.is_grad_enabled())
                if yr:
                    y = yr[0]
                m = layer.mlp(n)
                if drop is not None:
                    m = drop(m)
                outs.append(y + layer.post_feedforward_layernorm(m)[0])
                continue
            if g1 is None and drop is None:
                y = layer.self_attn.o_proj(a, residual=x)
            elif drop is None:
                op = layer.self_attn.o_proj
                y = ops.linear_gated_residual(a.to(op.weight.dtype), op.weight, op.bias, x, g1)
            else:
                y = ops.dropout_gated_residual(x, layer.self_attn.o_proj(a), g1, drop.p, True)
            fork = torch.is_grad_enabled()
            if mods[ti] is not None:
                n, g2, *yr = layer.post_attention_layernorm(y, precomputed=mods[ti][2 * li + 1], fork=fork)
            else:
                n, g2, *yr = layer.post_attention_layernorm(y, fork=fork)
            if yr:
                y = yr[0]
            if g2 is None and drop is None:
                outs.append(layer.mlp(n, residual=y))
            elif drop is None:
                mlp = layer.mlp
                outs.append(ops.gated_mlp_gated_residual(n.to(mlp.gate_up_proj.weight.dtype), mlp.gate_up_proj.weight,
                                                         mlp.down_proj.weight, mlp.act, y, g2))
            else:
                outs.append(ops.dropout_gated_residual(y, layer.mlp(n), g2, drop.p, True))
        return outs, new_k, new_v

    def forward(self, inputs_embeds: list[Tensor | None], position_ids: Tensor, q_blk: Tensor,
                q_valid: Tensor, *, adarms_cond: list[Tensor | None] | None = None,
                past: KVCache | None = None, fill_cache_len: int | None = None,
                k_blk: Tensor | None = None, k_valid: Tensor | None = None,
                mrope: bool = False, per_layer_cache: bool = True, past_layer_map: list[int] | None = None,
                layer_hook=None, cache_room: int = 0, cp=None) -> tuple[list[Tensor | None], KVCache | None]:
        """One pass over all layers.

        ``position_ids``: ``(B, S_total)`` (or ``(3,B,S_total)`` with ``mrope``) for the
        concatenated present towers.  ``q_blk/q_valid`` describe those tokens; when ``past`` is
        given its tokens are prepended as keys with block id ``INT_MIN`` (visible to every
        query, gated only by ``past.valid``).  ``fill_cache_len=n`` returns a cache holding the
        first ``n`` tokens' post-RoPE K/V of every layer.  ``past_layer_map[l]`` names the cache layer that
        decoder layer ``l`` reads (default ``l``; a constant map conditions every layer on one backbone
        layer).  ``layer_hook(l, xs) -> xs`` runs after layer ``l`` (deepstack feature injection).
        ``cache_room`` allocates the returned cache with that many spare token slots, so that a later
        single-tower inference pass can append its keys / values in place instead of concatenating.
        ``cp`` (a :class:`opentau_b200.parallel.cp.ContextParallel`): the tokens given are this rank's slice of
        every sequence; ``k_blk / k_valid`` must then describe the keys of ALL ranks (rank-major), attention runs
        across the ranks, and a filled cache holds this rank's keys / values only.
        """
        if cp is not None and (past is not None or k_blk is None):
            raise ValueError("a context-parallel pass needs the block ids of all keys and takes no cached prefix")
        cp = cp if (cp is not None and cp.world > 1) else None
        towers = self.towers
        xs = list(inputs_embeds)
        present = [t for t, x in zip(towers, xs) if x is not None]
        hd = present[0].cfg.head_dim
        adarms_cond = adarms_cond or [None] * len(towers)
        mods = [self._ada_mods(t, c) if x is not None else None for t, c, x in zip(towers, adarms_cond, xs)]

        if k_blk is None:
            k_blk, k_valid = q_blk, q_valid
        if past is not None:
            B = q_blk.shape[0]
            cross_blk = torch.full((B, past.length), ops.INT_MIN, dtype=torch.int32, device=q_blk.device)
            k_blk = torch.cat([cross_blk, k_blk], dim=1)
            k_valid = torch.cat([past.valid[:, :past.length], k_valid], dim=1)

        # RoPE tables once per distinct base (Gemma-3 alternates two bases across layers).
        table_cache: dict[float, tuple[Tensor, Tensor]] = {}

        def tables(theta: float):
            if theta not in table_cache:
                if mrope:
                    table_cache[theta] = ops.mrope_angles(position_ids, hd, theta, True,
                                                          present[0].cfg.mrope_sections)
                else:
                    table_cache[theta] = ops.rope_angles(position_ids, hd, theta)
            return table_cache[theta]

        new_cache = None
        if fill_cache_len is not None:
            B = q_blk.shape[0]
            hk = present[0].cfg.num_key_value_heads
            ref_x = next(x for x in xs if x is not None)
            new_cache = KVCache(
                ref_x.new_empty(self.num_layers, B, fill_cache_len + cache_room, hk, hd),
                ref_x.new_empty(self.num_layers, B, fill_cache_len + cache_room, hk, hd),
                q_valid[:, :fill_cache_len], fill_cache_len)
        keep_graph = fill_cache_len is not None and torch.is_grad_enabled()
        ks_list, vs_list = [], []
        live = [x for x in xs if x is not None]
        T_new = sum(x.shape[1] for x in live)
        one_tower_inference = len(live) == 1 and ops.can_fuse_qkv_post(live[0], hd)
        # in-place K/V: append behind the cached prefix (room permitting), or write a fresh cache directly
        append_in_place = one_tower_inference and past is not None and past.writable_room() >= T_new
        fill_in_place = (one_tower_inference and past is None and fill_cache_len is not None and not keep_graph
                         and fill_cache_len == T_new)

        gate = self.param_gate
        for li in range(self.num_layers):
            units = gate.enter([t.layers[li] for t, x in zip(towers, xs) if x is not None]) if gate is not None else None
            theta = towers[0].cfg.layer_theta(li)
            pl = past_layer_map[li] if past_layer_map is not None else li
            ck = past.k[pl, :, :past.length] if past is not None else None
            cv = past.v[pl, :, :past.length] if past is not None else None
            if self.gradient_checkpointing and self.training and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint
                xs, nk, nv = checkpoint(self._layer, li, xs, tables(theta), q_blk, k_blk, q_valid, k_valid,
                                        ck, cv, mods, None, cp, use_reentrant=False)
            else:
                kv_dst = None
                if append_in_place:
                    kv_dst = (past.k[pl], past.v[pl], past.length)
                elif fill_in_place:
                    kv_dst = (new_cache.k[li], new_cache.v[li], 0)
                xs, nk, nv = self._layer(li, xs, tables(theta), q_blk, k_blk, q_valid, k_valid, ck, cv, mods, kv_dst,
                                         cp)
            if units:
                xs = gate.leave(xs, units)
                if nk is not None and nk.requires_grad:       # keys / values that feed a later pass carry gradients too
                    nk, nv = gate.leave([nk, nv], units)
            if layer_hook is not None:
                xs = layer_hook(li, xs)
            if fill_cache_len is not None and not fill_in_place:
                if keep_graph:
                    ks_list.append(nk[:, :fill_cache_len])
                    vs_list.append(nv[:, :fill_cache_len])
                else:
                    new_cache.k[li, :, :fill_cache_len].copy_(nk[:, :fill_cache_len])
                    new_cache.v[li, :, :fill_cache_len].copy_(nv[:, :fill_cache_len])
        if keep_graph:
            new_cache = KVCache(torch.stack(ks_list), torch.stack(vs_list), new_cache.valid, fill_cache_len)

        outs: list[Tensor | None] = []
        for ti, (tower, x) in enumerate(zip(towers, xs)):
            if x is None:
                outs.append(None)
            elif mods[ti] is not None:
                outs.append(tower.norm(x, precomputed=mods[ti][2 * self.num_layers])[0])
            else:
                outs.append(tower.norm(x)[0])
        return outs, new_cache
