"""Context parallelism: block-causal attention over a sequence that is sharded across the ranks of one node.

The reference has no sequence / context parallelism (its longest-context tool is a single-GPU sweep,
``src/opentau/scripts/benchmark_flash_attn.py:329-388``); the pi0.7 configuration with 16 frames x 3 cameras
(12 288 vision tokens per sample) is where one GPU's activations and attention time stop being comfortable.

Layout: every rank holds a contiguous ``Sl = S / W`` slice of each sample's tokens and computes q/k/v for it.  The
forward pass is ONE kernel per rank (``ops/csrc/attention_cp_tcgen05.cu``): copier CTAs pull all ranks' K/V shards
over NVLink into a local gathered buffer exactly once, in ring order starting with the own shard, while the
attention CTAs (tcgen05 / TMEM flash attention) consume key blocks as they land.  Block ids / validity of ALL keys
are an input on every rank (they derive from the batch layout, which is replicated), in source-major order.

The backward pass keeps everything query-sided (q, dO, O, LSE) local, so its memory scales with 1 / W: every rank
gathers K / V of all ranks (peer loads into a local buffer; with grouped-query attention they are the small
tensors), runs ONE backward over its own queries against all keys -- which yields dQ of its queries and its
contribution to dK / dV of every key -- and the dK / dV contributions go back to the ranks that own the keys by a
reduce-scatter over peer memory that sums in rank order (deterministic).  No query, output or gradient-of-output
tensor ever leaves its rank.

``seq_scatter`` / ``seq_gather`` switch a batch between "my samples, whole sequences" and "all samples of the
group, my slice of every sequence" with an all-to-all (and its transpose in the backward pass): the vision encoder
and the loss heads work per sample, the decoder layers per sequence slice.

``backend="dist"`` (CPU / gloo, and the baseline the fused kernel is measured against) all-gathers K/V with the
library and calls the ordinary attention op.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p

import torch
import torch.distributed as dist
from torch import Tensor

MAX_RANKS = 8
DEFAULT_WAIT_BUDGET = 20_000_000_000


def _ptr_array(ptrs: list[int]):
    return (c_void_p * MAX_RANKS)(*[c_void_p(p) for p in ptrs], *[c_void_p(0)] * (MAX_RANKS - len(ptrs)))


class _Site:
    def __init__(self, ctx: "ContextParallel", B: int, Sl: int, Hkv: int, D: int):
        W = ctx.world
        self.numel = B * Sl * Hkv * D
        self.k = ctx._alloc(2 * self.numel * 2)            # two parities of this rank's K shard
        self.v = ctx._alloc(2 * self.numel * 2)
        self.ready = ctx._alloc(4 * MAX_RANKS, zero=True)
        self.kg = torch.empty(W * self.numel, dtype=torch.bfloat16, device=ctx.device)
        self.vg = torch.empty(W * self.numel, dtype=torch.bfloat16, device=ctx.device)
        bn = int(ctx.lib.otb_attn_cp_block(c_int(D)))
        self.gcount = torch.zeros(W * B * ((Sl + bn - 1) // bn + 1) + 1, dtype=torch.int32, device=ctx.device)
        self.epoch = 0
        # one copier CTA moves 10-30 GB/s (its shared memory bounds the bytes in flight): one per MB of remote K/V,
        # between 4 and 32
        remote_mb = (W - 1) * 2 * self.numel * 2 >> 20
        self.copiers = ctx.num_copiers or min(32, max(4, remote_mb))

    def ptrs(self, buf, parity: int) -> list[int]:
        return [p + parity * self.numel * 2 for p in buf.peer_ptrs]

    def local(self, buf, parity: int) -> Tensor:
        return buf.view(torch.bfloat16, 2 * self.numel)[parity * self.numel:(parity + 1) * self.numel]


class ContextParallel:
    def __init__(self, device, group=None, backend: str = "auto", num_copiers: int | None = None,
                 wait_budget: int = DEFAULT_WAIT_BUDGET):
        self.device = torch.device(device)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > MAX_RANKS:
            raise ValueError(f"context parallelism spans at most {MAX_RANKS} ranks of one node")
        if backend == "auto":
            backend = "p2p" if self.device.type == "cuda" else "dist"
        self.backend, self.num_copiers, self.wait_budget = backend, num_copiers, wait_budget
        self._sites: dict[tuple, _Site] = {}
        self._bufs: list = []
        if backend == "p2p":
            from ..ops import _lib, cuda_ops
            self.lib = _lib.load("attention_cp_tcgen05")
            self.comm_lib = _lib.load("comm_p2p")
            self.status = cuda_ops.status_pointer()

    def _alloc(self, nbytes: int, zero: bool = False):
        from .comm import SymmetricBuffer
        buf = SymmetricBuffer(self.comm_lib, max(nbytes, 256), self.device, self.group)
        if zero:
            buf.bytes_tensor.zero_()
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
        self._bufs.append(buf)
        return buf

    def shard(self, x: Tensor, dim: int = 1) -> Tensor:
        """This rank's contiguous slice of a full-sequence tensor along ``dim``."""
        n = x.shape[dim]
        if n % self.world:
            raise ValueError(f"sequence length {n} is not divisible by {self.world} ranks")
        per = n // self.world
        return x.narrow(dim, self.rank * per, per)

    def all_gather_seq(self, x: Tensor, dim: int = 1) -> Tensor:
        """Library all-gather along the sequence axis (source-major order)."""
        if self.world == 1:
            return x
        parts = [torch.empty_like(x) for _ in range(self.world)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.cat(parts, dim)

    # -- forward ------------------------------------------------------------------------------------------
    def attention_forward(self, q: Tensor, k: Tensor, v: Tensor, q_blk: Tensor, k_blk_all: Tensor, q_valid: Tensor,
                          k_valid_all: Tensor, scale: float) -> tuple[Tensor, Tensor]:
        """``q (B,Sl,H,D)``, ``k, v (B,Sl,Hkv,D)`` local; ``k_blk_all / k_valid_all (B, W*Sl)`` for all keys.
        Returns ``o (B, Sl, H*D)`` and ``lse (B, H, Sl)``."""
        B, Sl, H, D = q.shape
        Hkv = k.shape[2]
        if self.backend == "dist":
            from ..ops import prims
            kf, vf = self.all_gather_seq(k), self.all_gather_seq(v)
            return prims.attn_fwd(q, kf, vf, q_blk, k_blk_all, q_valid, k_valid_all, scale)
        from ..ops import cuda_ops
        key = (B, Sl, Hkv, D)
        if key not in self._sites:
            self._sites[key] = _Site(self, *key)
        site = self._sites[key]
        site.epoch += 1
        par = site.epoch & 1
        site.local(site.k, par).view(B, Sl, Hkv, D).copy_(k)
        site.local(site.v, par).view(B, Sl, Hkv, D).copy_(v)
        rc = self.lib.otb_cp_publish(_ptr_array(site.ready.peer_ptrs), c_int(self.rank), c_int(self.world),
                                     c_uint(site.epoch), self._stream())
        if rc != 0:
            raise RuntimeError(f"publish launch failed ({rc})")
        if q.stride(-1) != 1 or any(s % 8 for s in q.stride()[:3]) or q.data_ptr() % 16:
            q = q.contiguous()
        o = torch.empty(B, Sl, H, D, dtype=torch.bfloat16, device=self.device)
        lse = torch.empty(B, H, Sl, dtype=torch.float32, device=self.device)
        qb, kb = q_blk.to(torch.int32).contiguous(), k_blk_all.to(torch.int32).contiguous()
        qv, kv = q_valid.to(torch.uint8).contiguous(), k_valid_all.to(torch.uint8).contiguous()
        rc = self.lib.otb_attn_fwd_cp(
            c_void_p(q.data_ptr()), c_void_p(o.data_ptr()), c_void_p(lse.data_ptr()), c_void_p(qb.data_ptr()),
            c_void_p(kb.data_ptr()), c_void_p(qv.data_ptr()), c_void_p(kv.data_ptr()), c_int(B), c_int(Sl), c_int(Sl),
            c_int(H), c_int(Hkv), c_int(D), c_longlong(q.stride(0)), c_longlong(q.stride(1)), c_longlong(q.stride(2)),
            _ptr_array(site.ptrs(site.k, par)), _ptr_array(site.ptrs(site.v, par)), c_void_p(site.kg.data_ptr()),
            c_void_p(site.vg.data_ptr()), c_void_p(site.gcount.data_ptr()), c_void_p(site.ready.local_ptr),
            c_int(self.rank), c_int(self.world), c_uint(site.epoch), c_int(site.copiers), c_float(scale),
            c_longlong(self.wait_budget), c_void_p(self.status), self._stream())
        if rc != 0:
            raise RuntimeError(f"context-parallel attention launch failed ({rc})")
        cuda_ops.launch_count += 2
        self._last_site = site
        return o.view(B, Sl, H * D), lse

    def _stream(self) -> c_void_p:
        return c_void_p(torch.cuda.current_stream().cuda_stream)

    # -- sequence <-> sample layouts -------------------------------------------------------------------------
    def seq_scatter(self, x: Tensor) -> Tensor:
        """``(B, S, ...)`` for this rank's ``B`` samples -> ``(W * B, S / W, ...)``: this rank's slice of every
        sample of the group (rank-major sample order).  Differentiable."""
        return _SeqExchange.apply(self, x, True) if self.world > 1 else x

    def seq_gather(self, x: Tensor) -> Tensor:
        """Inverse of :meth:`seq_scatter`.  Differentiable."""
        return _SeqExchange.apply(self, x, False) if self.world > 1 else x

    def _exchange(self, x: Tensor, scatter: bool) -> Tensor:
        W = self.world
        if scatter:
            B, S = x.shape[:2]
            if S % W:
                raise ValueError(f"sequence length {S} is not divisible by {W} ranks")
            send = x.reshape(B, W, S // W, *x.shape[2:]).transpose(0, 1).contiguous()      # (W, B, Sl, ...)
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send, group=self.group)
            return recv.reshape(W * B, S // W, *x.shape[2:])
        WB, Sl = x.shape[:2]
        B = WB // W
        send = x.reshape(W, B, Sl, *x.shape[2:]).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)                               # recv[j] = slice j
        return recv.transpose(0, 1).reshape(B, W * Sl, *x.shape[2:])

    def batch_all_gather(self, x: Tensor, dim: int = 0) -> Tensor:
        """Concatenates every rank's tensor along ``dim`` (rank-major): masks / ids of all samples of the group."""
        if self.world == 1:
            return x
        parts = [torch.empty_like(x) for _ in range(self.world)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.cat(parts, dim)

    # -- backward data movement ------------------------------------------------------------------------------
    def _bwd_site(self, numel: int):
        """Symmetric staging for the backward pass of one K/V shape: this rank's K and V (gathered by peers) and
        its dK / dV contributions for all keys (reduced by their owners), two parities each."""
        key = ("bwd", numel)
        if key not in self._sites:
            W = self.world
            site = type("BwdSite", (), {})()
            site.kv = self._alloc(2 * 2 * numel * 2)                # [parity][k|v][numel] bf16
            site.dkv = self._alloc(2 * 2 * W * numel * 2)           # [parity][dk|dv][W * numel] bf16
            site.flags = self._alloc(4 * MAX_RANKS * 2, zero=True)  # slot 0: K/V staged, slot 1: dK/dV staged
            site.epoch = 0
            self._sites[key] = site
        return self._sites[key]

    def _barrier(self, site, slot: int) -> None:
        rc = self.comm_lib.otb_comm_barrier(_ptr_array(site.flags.peer_ptrs), c_int(self.rank), c_int(self.world),
                                            c_int(slot), c_int(site.epoch), c_longlong(self.wait_budget),
                                            c_void_p(self.status), self._stream())
        if rc != 0:
            raise RuntimeError(f"barrier launch failed ({rc})")

    def gather_kv(self, k: Tensor, v: Tensor):
        """K / V of all ranks, sequence-concatenated in rank order: ``(B, W * Sl, Hkv, D)`` each."""
        if self.world == 1:
            return k, v, None
        if self.backend == "dist":
            return self.all_gather_seq(k), self.all_gather_seq(v), None
        from ..ops import cuda_ops
        W, n = self.world, k.numel()
        site = self._bwd_site(n)
        site.epoch += 1
        par = site.epoch & 1
        stage = site.kv.view(torch.bfloat16, 4 * n)[par * 2 * n:(par + 1) * 2 * n]
        stage[:n].view(k.shape).copy_(k)
        stage[n:].view(v.shape).copy_(v)
        self._barrier(site, 0)
        out = torch.empty(W, 2, *k.shape, dtype=torch.bfloat16, device=self.device)
        src = [p + par * 2 * n * 2 for p in site.kv.peer_ptrs]
        rc = self.comm_lib.otb_comm_allgather_pull(_ptr_array(src), c_int(W), c_longlong(2 * n * 2),
                                                   c_void_p(out.data_ptr()), c_int(296), c_void_p(self.status),
                                                   self._stream())
        if rc != 0:
            raise RuntimeError(f"all-gather launch failed ({rc})")
        cuda_ops.launch_count += 2
        B, Sl = k.shape[:2]
        # (W, B, Sl, ...) -> (B, W * Sl, ...)
        kf = out[:, 0].transpose(0, 1).reshape(B, W * Sl, *k.shape[2:])
        vf = out[:, 1].transpose(0, 1).reshape(B, W * Sl, *k.shape[2:])
        return kf, vf, site

    def reduce_scatter_kv_grads(self, dkf: Tensor, dvf: Tensor, site) -> tuple[Tensor, Tensor]:
        """``dkf, dvf (B, W * Sl, Hkv, D)``: this rank's contributions for ALL keys -> the sums over ranks for the
        keys this rank owns, ``(B, Sl, Hkv, D)``."""
        W = self.world
        if W == 1:
            return dkf, dvf
        B, S = dkf.shape[:2]
        Sl = S // W
        tail = dkf.shape[2:]
        if self.backend == "dist":
            both = torch.stack([dkf, dvf]).float()
            dist.all_reduce(both, group=self.group)
            mine = both[:, :, self.rank * Sl:(self.rank + 1) * Sl]
            return mine[0].to(dkf.dtype).contiguous(), mine[1].to(dvf.dtype).contiguous()
        from ..ops import cuda_ops
        n = B * Sl * tail.numel()
        par = site.epoch & 1
        stage = site.dkv.view(torch.bfloat16, 4 * W * n)[par * 2 * W * n:(par + 1) * 2 * W * n]
        # owner-major: [dk | dv][owner][B, Sl, ...], so every owner's slice is one contiguous range
        stage[:W * n].view(W, B, Sl, *tail).copy_(dkf.reshape(B, W, Sl, *tail).transpose(0, 1))
        stage[W * n:].view(W, B, Sl, *tail).copy_(dvf.reshape(B, W, Sl, *tail).transpose(0, 1))
        self._barrier(site, 1)
        out = torch.empty(2, B, Sl, *tail, dtype=torch.bfloat16, device=self.device)
        src = [p + par * 2 * W * n * 2 for p in site.dkv.peer_ptrs]
        for which in range(2):
            rc = self.comm_lib.otb_comm_reduce_scatter_bf16(
                _ptr_array(src), c_int(W), c_longlong(which * W * n + self.rank * n), c_longlong(n),
                c_void_p(out[which].data_ptr()), c_int(296), c_void_p(self.status), self._stream())
            if rc != 0:
                raise RuntimeError(f"reduce-scatter launch failed ({rc})")
        cuda_ops.launch_count += 3
        return out[0], out[1]

    # -- autograd -------------------------------------------------------------------------------------------
    def attention(self, q: Tensor, k: Tensor, v: Tensor, q_blk: Tensor, k_blk_all: Tensor, q_valid: Tensor,
                  k_valid_all: Tensor, scale: float) -> Tensor:
        return _CPAttention.apply(self, q, k, v, q_blk, k_blk_all, q_valid, k_valid_all, scale)


class _CPAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, cp: ContextParallel, q, k, v, q_blk, k_blk_all, q_valid, k_valid_all, scale):
        o, lse = cp.attention_forward(q, k, v, q_blk, k_blk_all, q_valid, k_valid_all, scale)
        ctx.cp, ctx.scale = cp, scale
        ctx.save_for_backward(q, k, v, o, lse, q_blk, k_blk_all, q_valid, k_valid_all)
        return o

    @staticmethod
    def backward(ctx, do):
        from ..ops import prims
        cp: ContextParallel = ctx.cp
        q, k, v, o, lse, q_blk, k_blk_all, q_valid, k_valid_all = ctx.saved_tensors
        do = do.contiguous()
        kf, vf, site = cp.gather_kv(k, v)
        # own queries against all keys: dQ is final, dK / dV are this rank's contributions for every key
        dq, dkf, dvf = prims.attn_bwd(do, q, kf.contiguous(), vf.contiguous(), o, lse, q_blk, k_blk_all, q_valid,
                                      k_valid_all, ctx.scale)
        dk, dv = cp.reduce_scatter_kv_grads(dkf, dvf, site)
        return None, dq, dk.to(k.dtype), dv.to(v.dtype), None, None, None, None, None


class _SeqExchange(torch.autograd.Function):
    """All-to-all between the per-sample and the per-sequence-slice layout; the backward is the opposite exchange."""

    @staticmethod
    def forward(ctx, cp: ContextParallel, x, scatter: bool):
        ctx.cp, ctx.scatter = cp, scatter
        return cp._exchange(x, scatter)

    @staticmethod
    def backward(ctx, g):
        return None, ctx.cp._exchange(g.contiguous(), not ctx.scatter), None
