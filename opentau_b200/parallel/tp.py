"""Tensor parallelism with sequence-sharded activations, fused with its collectives over peer memory.

The reference has no tensor parallelism of its own (it shards with FSDP / DeepSpeed ZeRO through
``accelerate``: OpenTau ``src/opentau/scripts/train.py:728-737``, ``configs/examples/*zero*.yaml``); a frozen
32B-class backbone such as cosmos3's Qwen3-VL (``src/opentau/policies/cosmos3/qwen3vl_with_expert.py:115-207``)
is where a B200 box wants it.  Layout (Megatron sequence parallelism):

    x_local [M/W, d] --norm--> all-gather + column-parallel GEMM (qkv | gate_up) --> [M, n/W]
                     --attention on the local heads / GLU--> row-parallel GEMM + reduce-scatter --> [M/W, d]

Both collectives run INSIDE the GEMM kernels (``ops/csrc/gemm_dist_tcgen05.cu``): for the all-gather a copier
warp per CTA pulls the peers' rows over NVLink once (bulk async copies) while the tensor cores already work on
the rows that have landed; for the reduce-scatter the epilogue sends partial tiles with TMA stores into the
destination rank's staging buffer and the kernel's tail reduces them.  ``torch.distributed`` is used to exchange IPC
handles once, and as the CPU / fallback data path (``backend="dist"``), which is also the baseline the fused
kernels are measured against.

Rows are sharded in units of whole samples when ``M = B*S`` and ``B % W == 0``, so a rank's row shard is the
token range of its own samples.
"""

from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_uint, c_void_p

import torch
import torch.distributed as dist
from torch import Tensor

MAX_RANKS = 8
DEFAULT_WAIT_BUDGET = 20_000_000_000


def _ptr_array(ptrs: list[int]):
    return (c_void_p * MAX_RANKS)(*[c_void_p(p) for p in ptrs], *[c_void_p(0)] * (MAX_RANKS - len(ptrs)))


class _Site:
    """Peer-visible workspace of one call-site shape, double-buffered by step parity."""

    def __init__(self, ctx: "TensorParallel", kind: str, Ml: int, width: int):
        self.kind, self.Ml, self.width, self.epoch = kind, Ml, width, 0
        W = ctx.world
        if kind == "ag":
            self.numel = Ml * width                      # one parity of the activation shard [Ml, K]
            self.data = ctx._alloc(2 * self.numel * 2)
            self.sync = ctx._alloc(4 * MAX_RANKS, zero=True)   # ready[src]
            # private to this rank: the gathered rows and the piece counters / dispenser of the copier warps
            self.gathered = torch.empty(W * Ml, width, dtype=torch.bfloat16, device=ctx.device)
            self.gcount = torch.zeros(W * ((Ml + 127) // 128) + 1, dtype=torch.int32, device=ctx.device)
        else:
            self.numel = W * Ml * width                  # one parity of the staging [W, Ml, N]
            self.data = ctx._alloc(2 * self.numel * 2)
            self.sync = ctx._alloc(4 * W * ((Ml + 127) // 128), zero=True)  # counters[src][row block]

    def data_ptrs(self, parity: int) -> list[int]:
        return [p + parity * self.numel * 2 for p in self.data.peer_ptrs]

    def local(self, parity: int) -> Tensor:
        return self.data.view(torch.bfloat16, 2 * self.numel)[parity * self.numel:(parity + 1) * self.numel]


class TensorParallel:
    """Per-process tensor-parallel runtime (one per process group)."""

    def __init__(self, device, group=None, backend: str = "auto", wait_budget: int = DEFAULT_WAIT_BUDGET):
        self.device = torch.device(device)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > MAX_RANKS:
            raise ValueError(f"tensor parallelism spans at most {MAX_RANKS} ranks of one node")
        if backend == "auto":
            backend = "p2p" if self.device.type == "cuda" else "dist"
        self.backend = backend
        self.wait_budget = wait_budget
        self._sites: dict[tuple, _Site] = {}
        self._bufs: list = []
        if backend == "p2p":
            from ..ops import _lib, cuda_ops
            self.lib = _lib.load("gemm_dist_tcgen05")
            self.comm_lib = _lib.load("comm_p2p")
            self.status = cuda_ops.status_pointer()

    # -- workspaces -----------------------------------------------------------------------------------
    def _alloc(self, nbytes: int, zero: bool = False):
        from .comm import SymmetricBuffer
        buf = SymmetricBuffer(self.comm_lib, max(nbytes, 256), self.device, self.group)
        if zero:
            buf.bytes_tensor.zero_()
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
        self._bufs.append(buf)
        return buf

    def _site(self, kind: str, Ml: int, width: int, other: int) -> _Site:
        """Workspace of one call shape.  The in-kernel counters count monotonically and assume that every step on
        a site launches the same grid, so the key holds the complete GEMM shape."""
        key = (kind, Ml, width, other)
        if key not in self._sites:
            self._sites[key] = _Site(self, kind, Ml, width)
        return self._sites[key]

    def _stream(self) -> c_void_p:
        return c_void_p(torch.cuda.current_stream().cuda_stream)

    # -- sharding helpers -------------------------------------------------------------------------------
    def shard_rows(self, w: Tensor, unit: int = 1) -> Tensor:
        """Rank's contiguous block of output rows of ``w``; ``unit`` = indivisible group of rows."""
        n = w.shape[0]
        if n % (self.world * unit):
            raise ValueError(f"{n} rows cannot be split over {self.world} ranks in units of {unit}")
        per = n // self.world
        return w[self.rank * per:(self.rank + 1) * per].contiguous()

    def shard_cols(self, w: Tensor, unit: int = 1) -> Tensor:
        n = w.shape[1]
        if n % (self.world * unit):
            raise ValueError(f"{n} columns cannot be split over {self.world} ranks in units of {unit}")
        per = n // self.world
        return w[:, self.rank * per:(self.rank + 1) * per].contiguous()

    # -- all-gather -> GEMM -----------------------------------------------------------------------------
    def ag_buffer(self, Ml: int, K: int, N: int) -> Tensor:
        """The peer-visible ``[Ml, K]`` buffer the NEXT :meth:`all_gather_linear` of this shape reads; writing
        the activation straight into it (e.g. as a norm kernel's output) saves the staging copy."""
        site = self._site("ag", Ml, K, N)
        return site.local((site.epoch + 1) & 1).view(Ml, K)

    def all_gather_linear(self, x_local: Tensor, w: Tensor, bias: Tensor | None = None) -> Tensor:
        """``concat_r(x_r) @ w.T (+ bias)``: ``x_local [Ml, K]``, ``w [N_local, K]`` -> ``[W*Ml, N_local]``."""
        Ml, K = x_local.shape
        N = w.shape[0]
        if self.backend == "dist" or self.world == 1 and self.device.type != "cuda":
            if self.world > 1:
                parts = [torch.empty_like(x_local) for _ in range(self.world)]
                dist.all_gather(parts, x_local.contiguous(), group=self.group)
                x = torch.cat(parts, 0)
            else:
                x = x_local
            from .. import ops
            return ops.linear(x, w, bias)
        from ..ops import cuda_ops
        site = self._site("ag", Ml, K, N)
        site.epoch += 1
        par = site.epoch & 1
        buf = site.local(par).view(Ml, K)
        if x_local.data_ptr() != buf.data_ptr():
            buf.copy_(x_local)
        rc = self.lib.otb_dist_publish(_ptr_array(site.sync.peer_ptrs), c_int(self.rank), c_int(self.world),
                                       c_uint(site.epoch), self._stream())
        if rc != 0:
            raise RuntimeError(f"publish launch failed ({rc})")
        out = torch.empty(self.world * Ml, N, dtype=torch.bfloat16, device=self.device)
        rc = self.lib.otb_ag_gemm_bf16(
            _ptr_array(site.data_ptrs(par)), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), c_int(Ml), c_int(N),
            c_int(K), c_longlong(w.stride(0)), c_longlong(N), c_void_p(bias.data_ptr() if bias is not None else 0),
            c_void_p(site.sync.local_ptr), c_void_p(site.gathered.data_ptr()), c_void_p(site.gcount.data_ptr()),
            c_int(self.rank), c_int(self.world), c_uint(site.epoch), c_longlong(self.wait_budget),
            c_void_p(self.status), self._stream())
        if rc != 0:
            raise RuntimeError(f"all-gather GEMM launch failed ({rc})")
        cuda_ops.launch_count += 2
        return out

    def fsdp_linear(self, x: Tensor, w_shard: Tensor, bias: Tensor | None = None) -> Tensor:
        """Parameter-sharded (FSDP / ZeRO-3 style) linear: every rank owns ``w_shard [N/W, K]`` (consecutive output
        rows of the weight) and has its OWN activations ``x [M, K]``; returns ``x @ W_full^T (+ bias)`` as ``[M, N]``.

        The parameter all-gather is fused into the GEMM that consumes it: the weight shards are the gathered operand
        of the all-gather -> GEMM kernel (copier warps pull each peer's shard over NVLink once while the tensor-core
        tiles of shards that already arrived run), the local activations are the stationary operand, and the kernel
        produces ``W_full @ x^T``; the result is returned as its transposed view (call ``.contiguous()`` where a
        row-major tensor is required).  Nothing of the full weight outlives the call."""
        yt = self.all_gather_linear(w_shard, x)          # [N, M]
        y = yt.t()
        return y + bias if bias is not None else y

    # -- GEMM -> reduce-scatter -------------------------------------------------------------------------
    def linear_reduce_scatter(self, x: Tensor, w: Tensor, bias: Tensor | None = None,
                              residual: Tensor | None = None) -> Tensor:
        """``sum_r(x_r @ w_r.T)`` scattered by rows: ``x [W*Ml, K_local]``, ``w [N, K_local]`` -> ``[Ml, N]``
        (+ ``bias`` once, + ``residual [Ml, N]``)."""
        M, Kl = x.shape
        N = w.shape[0]
        W = self.world
        if M % W:
            raise ValueError(f"{M} rows cannot be scattered over {W} ranks")
        Ml = M // W
        if self.backend == "dist" or W == 1 and self.device.type != "cuda":
            from .. import ops
            part = ops.linear(x, w)
            if W > 1:
                full = part.float()
                dist.all_reduce(full, group=self.group)
                part = full[self.rank * Ml:(self.rank + 1) * Ml].to(x.dtype)
            if bias is not None:
                part = part + bias
            return part + residual if residual is not None else part
        from ..ops import cuda_ops
        site = self._site("rs", Ml, N, Kl)
        site.epoch += 1
        par = site.epoch & 1
        x = x if x.is_contiguous() else x.contiguous()
        out = torch.empty(Ml, N, dtype=torch.bfloat16, device=self.device)
        rc = self.lib.otb_gemm_rs_bf16(
            c_void_p(x.data_ptr()), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), c_int(Ml), c_int(N), c_int(Kl),
            c_longlong(x.stride(0)), c_longlong(w.stride(0)), c_longlong(N),
            c_void_p(bias.data_ptr() if bias is not None else 0),
            c_void_p(residual.data_ptr() if residual is not None else 0),
            c_longlong(residual.stride(0) if residual is not None else 0), _ptr_array(site.data_ptrs(par)),
            _ptr_array(site.sync.peer_ptrs), c_int(self.rank), c_int(W), c_uint(site.epoch), c_int(3),
            c_longlong(self.wait_budget), c_void_p(self.status), self._stream())
        if rc != 0:
            raise RuntimeError(f"GEMM reduce-scatter launch failed ({rc})")
        cuda_ops.launch_count += 1
        return out


# ------------------------------------------------------------------------------------ a sharded decoder layer
class TPDecoderLayer(torch.nn.Module):
    """Inference-time tensor-parallel view of one :class:`~opentau_b200.models.layers.DecoderLayer`.

    Holds this rank's shard of the fused qkv / gate-up / o / down weights (heads and MLP columns split over the
    ranks; KV heads are replicated when there are fewer of them than ranks) and runs the layer on a
    sequence-sharded hidden state.  Built for frozen backbones: weights are plain buffers.
    """

    def __init__(self, layer, tp: TensorParallel):
        super().__init__()
        cfg = layer.cfg
        W, r = tp.world, tp.rank
        self.tp, self.cfg = tp, cfg
        H, Hk, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        if H % W:
            raise ValueError(f"{H} attention heads cannot be split over {W} ranks")
        self.h_local = H // W
        self.kv_rep = max(1, W // Hk)                 # ranks sharing one KV head
        self.hk_local = max(1, Hk // W)
        if Hk >= W and Hk % W:
            raise ValueError(f"{Hk} KV heads cannot be split over {W} ranks")
        wq, wk, wv = layer.self_attn.qkv_proj.weight.detach().split([H * D, Hk * D, Hk * D], dim=0)
        q = wq[r * self.h_local * D:(r + 1) * self.h_local * D]
        k0 = (r // self.kv_rep) * self.hk_local if Hk < W else r * self.hk_local
        k = wk[k0 * D:(k0 + self.hk_local) * D]
        v = wv[k0 * D:(k0 + self.hk_local) * D]
        self.register_buffer("w_qkv", torch.cat([q, k, v], 0).contiguous(), persistent=False)
        self.register_buffer("w_o", tp.shard_cols(layer.self_attn.o_proj.weight.detach(), D), persistent=False)
        self.register_buffer("w_gu", tp.shard_rows(layer.mlp.gate_up_proj.weight.detach(), 64), persistent=False)
        self.register_buffer("w_down", tp.shard_cols(layer.mlp.down_proj.weight.detach(), 32), persistent=False)
        self.act = layer.mlp.act
        self.input_layernorm = layer.input_layernorm
        self.post_attention_layernorm = layer.post_attention_layernorm
        self.q_norm = getattr(layer.self_attn, "q_norm", None)
        self.k_norm = getattr(layer.self_attn, "k_norm", None)

    def forward(self, x_local: Tensor, B: int, S: int, cos_sin, blk: Tensor, valid: Tensor):
        """``x_local [B*S/W, d]`` -> ``(x_local', k, v)`` with ``k, v [B, S, hk_local, D]`` (post-RoPE) of the
        local heads.  ``cos_sin``/``blk``/``valid`` describe the FULL ``[B, S]`` sequence."""
        from .. import ops
        tp, D = self.tp, self.cfg.head_dim
        h = self.input_layernorm(x_local)[0]
        qkv = tp.all_gather_linear(h, self.w_qkv)
        q, k, v = qkv.view(B, S, -1).split([self.h_local * D, self.hk_local * D, self.hk_local * D], dim=-1)
        q, k, v = q.unflatten(-1, (self.h_local, D)), k.unflatten(-1, (self.hk_local, D)), v.unflatten(-1, (self.hk_local, D))
        if self.q_norm is not None:
            q, k = self.q_norm(q)[0], self.k_norm(k)[0]
        q, k = ops.rope(q, *cos_sin), ops.rope(k, *cos_sin)
        att = ops.block_attention(q, k, v, blk, blk, valid, valid, self.cfg.attn_scale)
        y = tp.linear_reduce_scatter(att.reshape(B * S, -1), self.w_o, residual=x_local)
        n = self.post_attention_layernorm(y)[0]
        gu = tp.all_gather_linear(n, self.w_gu)
        hmid = ops.prims.glu_fwd(gu, self.act)
        out = tp.linear_reduce_scatter(hmid, self.w_down, residual=y)
        return out, k, v
