"""Building blocks shared by every model family: linear, norms, attention, gated MLP.

Module and parameter names follow the HuggingFace Gemma / SigLIP / Qwen3 naming so that the
state-dict keys match the reference checkpoints (``q_proj``, ``input_layernorm``,
``…layernorm.dense.{weight,bias}`` for adaptive norms — see OpenTau
``src/opentau/utils/transformers_patch.py:92-167``).  The math lives in ``opentau_b200.ops``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from .. import ops


class Linear(nn.Module):
    """``nn.Linear``-compatible parameters; forward goes through ``ops.linear`` (tcgen05 GEMM)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False,
                 dtype: torch.dtype | None = None, zero_init: bool = False):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype)) if bias else None
        if zero_init:
            nn.init.zeros_(self.weight)
        else:
            nn.init.normal_(self.weight, std=0.02)

    def forward(self, x: Tensor, residual: Tensor | None = None) -> Tensor:
        w, b = self.weight, self.bias
        if x.dtype != w.dtype:
            x = x.to(w.dtype)
        pad_o, pad_i = -self.out_features % 8, -self.in_features % 8
        if (pad_o or pad_i) and x.is_cuda:
            # the tensor-core path moves rows of 16 bytes: widths that are not a multiple of 8 (a 201-bin value head)
            # run on zero-padded copies; autograd slices the gradients back
            w = F.pad(w, (0, pad_i, 0, pad_o))
            b = F.pad(b, (0, pad_o)) if b is not None else None
            x = F.pad(x, (0, pad_i)) if pad_i else x
            y = ops.linear(x, w, b)[..., :self.out_features]
            return y + residual if residual is not None else y
        return ops.linear(x, w, b, residual)

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}"


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, unit_offset: bool = True):
        super().__init__()
        self.eps, self.unit_offset = eps, unit_offset
        self.weight = nn.Parameter(torch.zeros(dim) if unit_offset else torch.ones(dim))

    def forward(self, x: Tensor, cond: Tensor | None = None, fork: bool = False):
        """``(y, None)``; with ``fork`` ``(y, None, x_res)`` where ``x_res`` carries ``x`` to the residual connection
        around this norm's branch (``ops.rms_norm_fork``)."""
        if fork:
            y, xr = ops.rms_norm_fork(x, self.weight, self.eps, self.unit_offset)
            return y, None, xr
        return ops.rms_norm(x, self.weight, self.eps, self.unit_offset), None


class AdaRMSNorm(nn.Module):
    """RMSNorm whose scale/shift/gate come from ``dense(cond)``; the dense layer is zero-init.

    ``precomputed`` lets the caller hand in ``dense(cond)`` computed for all layers in one GEMM
    (the condition does not change from layer to layer).
    """

    def __init__(self, dim: int, cond_dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps, self.dim = eps, dim
        self.dense = Linear(cond_dim, 3 * dim, bias=True, zero_init=True)

    def forward(self, x: Tensor, cond: Tensor | None = None, precomputed: Tensor | None = None, fork: bool = False):
        if precomputed is None:
            if cond is None:
                raise ValueError("AdaRMSNorm needs a condition")
            precomputed = self.dense(cond.to(self.dense.weight.dtype))
        if fork:
            return ops.ada_rms_norm_fork(x, precomputed, self.eps)
        return ops.ada_rms_norm(x, precomputed, self.eps)


class LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))
        self.bias = nn.Parameter(torch.zeros(dim))

    def forward(self, x: Tensor) -> Tensor:
        return ops.layer_norm(x, self.weight, self.bias, self.eps)


@dataclass
class TowerConfig:
    """Geometry of one decoder tower (a VLM text backbone or an action expert)."""

    hidden_size: int = 2048
    num_hidden_layers: int = 18
    num_attention_heads: int = 8
    num_key_value_heads: int = 1
    head_dim: int = 256
    intermediate_size: int = 16384
    vocab_size: int = 257152
    hidden_act: str = "gelu_tanh"          # "gelu_tanh" (Gemma GeGLU) | "silu" (Qwen SwiGLU)
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_local_theta: float | None = None  # Gemma-3 sliding layers
    sliding_window_pattern: int = 0        # every pattern-th layer is global; 0 = all global
    norm_unit_offset: bool = True          # Gemma (1+w)
    use_adarms: bool = False
    adarms_cond_dim: int | None = None
    adarms_has_weight: bool = False
    qk_norm: bool = False                  # per-head RMSNorm on q and k before RoPE
    sandwich_norms: bool = False           # Gemma-3: post-attn / pre-ffw / post-ffw norms
    query_pre_attn_scalar: float | None = None
    attention_bias: bool = False
    embed_scale: bool = True               # multiply token embeddings by sqrt(hidden)
    mrope_sections: tuple[int, ...] | None = None

    @property
    def attn_scale(self) -> float:
        base = self.query_pre_attn_scalar if self.query_pre_attn_scalar is not None else self.head_dim
        return float(base) ** -0.5

    def layer_theta(self, layer_idx: int) -> float:
        if self.rope_local_theta is not None and self.sliding_window_pattern:
            is_global = (layer_idx + 1) % self.sliding_window_pattern == 0
            return self.rope_theta if is_global else self.rope_local_theta
        return self.rope_theta


def make_norm(cfg: TowerConfig, dim: int | None = None) -> nn.Module:
    dim = dim or cfg.hidden_size
    if cfg.use_adarms:
        return AdaRMSNorm(dim, cfg.adarms_cond_dim or dim, cfg.rms_norm_eps)
    return RMSNorm(dim, cfg.rms_norm_eps, cfg.norm_unit_offset)


class Attention(nn.Module):
    """Projections of one tower's attention; the score computation is shared across towers.

    q, k and v are one fused parameter ``qkv_proj.weight`` of shape ``((H+2Hkv)·D, d)`` so a single
    GEMM serves all three; ``state_dict`` still exposes/accepts ``q_proj / k_proj / v_proj`` keys.
    """

    def __init__(self, cfg: TowerConfig):
        super().__init__()
        self.cfg = cfg
        d, h, hk, hd = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        self.qkv_proj = Linear(d, (h + 2 * hk) * hd, bias=cfg.attention_bias)
        self.o_proj = Linear(h * hd, d, bias=cfg.attention_bias)
        if cfg.qk_norm:
            self.q_norm = RMSNorm(hd, cfg.rms_norm_eps, cfg.norm_unit_offset)
            self.k_norm = RMSNorm(hd, cfg.rms_norm_eps, cfg.norm_unit_offset)
        self._splits = [h * hd, hk * hd, hk * hd]
        self._register_state_dict_hook(_split_hook("qkv_proj", ["q_proj", "k_proj", "v_proj"], self._splits))
        self._register_load_state_dict_pre_hook(
            _merge_hook("qkv_proj", ["q_proj", "k_proj", "v_proj"]), with_module=False)

    def qkv(self, x: Tensor) -> tuple[Tensor, Tensor, Tensor]:
        """``x (B,S,d)`` -> q ``(B,S,H,D)``, k, v ``(B,S,Hkv,D)`` as strided views of one GEMM output."""
        cfg = self.cfg
        h, hk, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        out = self.qkv_proj(x)
        q, k, v = out.split(self._splits, dim=-1)
        q = q.unflatten(-1, (h, hd))
        k = k.unflatten(-1, (hk, hd))
        v = v.unflatten(-1, (hk, hd))
        if cfg.qk_norm:
            q = self.q_norm(q)[0]
            k = self.k_norm(k)[0]
        return q, k, v


def _split_hook(fused: str, names: list[str], sizes: list[int], interleaved: bool = False):
    """state_dict hook: replace ``<fused>.weight/bias`` by the per-projection entries."""

    def hook(module, state, prefix, local_metadata):
        for suffix in ("weight", "bias"):
            key = f"{prefix}{fused}.{suffix}"
            if key not in state:
                continue
            t = state.pop(key)
            if interleaved:
                if suffix == "weight":
                    parts = ops.prims.deinterleave_gate_up(t)
                else:
                    raise NotImplementedError
            else:
                parts = t.split(sizes, dim=0)
            for n, p in zip(names, parts):
                state[f"{prefix}{n}.{suffix}"] = p
        return state

    return hook


def _merge_hook(fused: str, names: list[str], interleaved: bool = False):
    """load_state_dict pre-hook: build ``<fused>.weight/bias`` from per-projection entries."""

    def hook(state, prefix, local_metadata, strict, missing, unexpected, errors):
        for suffix in ("weight", "bias"):
            keys = [f"{prefix}{n}.{suffix}" for n in names]
            if all(k in state for k in keys):
                parts = [state.pop(k) for k in keys]
                if interleaved:
                    state[f"{prefix}{fused}.{suffix}"] = ops.prims.interleave_gate_up(*parts)
                else:
                    state[f"{prefix}{fused}.{suffix}"] = torch.cat(parts, dim=0)

    return hook


class GatedMLP(nn.Module):
    """``down(act(gate(x)) * up(x))`` with gate and up fused into one block-interleaved weight
    (32 gate rows, 32 up rows, …) so the activation can run in the GEMM epilogue."""

    def __init__(self, cfg: TowerConfig):
        super().__init__()
        self.act = cfg.hidden_act
        self.gate_up_proj = Linear(cfg.hidden_size, 2 * cfg.intermediate_size)
        self.down_proj = Linear(cfg.intermediate_size, cfg.hidden_size)
        self._register_state_dict_hook(
            _split_hook("gate_up_proj", ["gate_proj", "up_proj"], [], interleaved=True))
        self._register_load_state_dict_pre_hook(
            _merge_hook("gate_up_proj", ["gate_proj", "up_proj"], interleaved=True), with_module=False)

    def forward(self, x: Tensor, residual: Tensor | None = None) -> Tensor:
        w = self.gate_up_proj.weight
        if x.dtype != w.dtype:
            x = x.to(w.dtype)
        return ops.gated_mlp(x, w, self.down_proj.weight, self.act, residual)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: TowerConfig, layer_idx: int):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.self_attn = Attention(cfg)
        self.mlp = GatedMLP(cfg)
        self.input_layernorm = make_norm(cfg)
        self.post_attention_layernorm = make_norm(cfg)
        if cfg.sandwich_norms:
            self.pre_feedforward_layernorm = make_norm(cfg)
            self.post_feedforward_layernorm = make_norm(cfg)


class Tower(nn.Module):
    """A stack of decoder layers with token embedding and final norm (``model`` in HF naming)."""

    def __init__(self, cfg: TowerConfig, with_embed: bool = True):
        super().__init__()
        self.cfg = cfg
        if with_embed:
            self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
            nn.init.normal_(self.embed_tokens.weight, std=0.02)
        self.layers = nn.ModuleList([DecoderLayer(cfg, i) for i in range(cfg.num_hidden_layers)])
        self.norm = make_norm(cfg)

    def embed(self, tokens: Tensor) -> Tensor:
        scale = math.sqrt(self.cfg.hidden_size) if self.cfg.embed_scale else 1.0
        return ops.embedding(self.embed_tokens.weight, tokens, scale)
