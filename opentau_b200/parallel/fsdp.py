"""Parameter-sharded data parallelism (``strategy = fsdp | fsdp2 | zero3``).

The reference reaches this through accelerate: FSDP1 / FSDP2 with wrap units ``InterleavedDecoderLayer`` and
``SiglipEncoderLayer`` (``configs/examples/accelerate_fsdp_config.yaml:16-33``) or DeepSpeed ZeRO-3
(``accelerate_deepspeed_zero3_config.yaml``); only the Gemma-3 family is wired for it there
(``scripts/train.py:902-916``).  Here it is one engine for every family:

* At rest every rank holds 1 / W of every parameter bucket as bf16 (``pshard``, in symmetric memory so peers can
  read it), next to its fp32 masters and Adam moments.  The full-size flat parameter buffer of the replicated
  strategies does not exist.
* A bucket is a UNIT: all parameters of one decoder layer of one tower (the two towers of an interleaved layer are
  two units, because a pass with one tower absent must not gather the other's weights), or "root" for what is used
  outside the layer loop (embeddings, heads, projector, the stacked adaptive-norm projections, a trained vision
  tower).  Root units are gathered once per step and stay; layer units are gathered right before the layer runs
  into one of two rotating slots per tower, and again (into the SAME slot, so tensors saved for the backward pass
  point at the right weights) right before the layer's backward.
* The gather is a kernel of ours: every rank pulls the W slices from its peers' ``pshard`` with plain loads over
  NVLink (``comm_p2p.cu: allgather_pull_kernel``); no flags are needed, the shards only change in the optimizer
  step, which ends with a barrier.  With the library backend (CPU / gloo, or ``comm="nccl"``) it is an all-gather.
* Gradients: as in ZeRO-2, each unit's gradient bucket is reduce-scattered to the owners of its slices as soon as
  the unit's backward has been issued; the sharded AdamW then writes the new bf16 values into the local ``pshard``
  only (no parameter all-gather in the optimizer step at all).

The all-gather fused INTO the product that consumes the shard (``parallel/tp.py: fsdp_linear`` on
``gemm_dist_tcgen05.cu``) covers a single linear whose weight is sharded by rows; units here are sliced as flat
ranges (a slice crosses parameter boundaries), so the engine gathers with the pull kernel.
"""

from __future__ import annotations

import re
from contextlib import contextmanager
from ctypes import c_int, c_longlong, c_void_p

import torch
import torch.distributed as dist
from torch import Tensor, nn

from .engine import OptimHyper, TrainEngine, _ShardState  # noqa: F401
from .flat import FlatParamStore

_LAYER = re.compile(r"(?:^|\.)(?P<stem>[A-Za-z0-9_.]*?)layers\.(?P<idx>\d+)\.(?P<rest>.*)$")


def unit_key(name: str) -> str:
    """Bucket key of a parameter: ``"<tower path>#<layer>"`` for a decoder layer's own weights, ``"root"`` for
    everything used outside the decoder's layer loop."""
    if ".dense." in name and "norm" in name:            # adaptive-norm projections: one stacked product up front
        return "root"
    if "vision" in name or "video_encoder" in name:
        return "root"
    m = _LAYER.search(name)
    if m is None:
        return "root"
    rest = m.group("rest")
    tower = name[: m.start("idx")]
    if rest.startswith("backbone_layer."):              # Gemma-3 interleaved layout: one module, two towers
        tower += "backbone"
    elif rest.startswith("expert_layer."):
        tower += "expert"
    return f"{tower}#{int(m.group('idx'))}"


class _BackwardAcquire(torch.autograd.Function):
    """Identity whose backward makes a unit resident: placed on a layer's OUTPUT, it runs before every backward
    kernel (and before any recomputation) of that layer."""

    @staticmethod
    def forward(ctx, x, gate, unit):
        ctx.gate, ctx.unit = gate, unit
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.gate.acquire(ctx.unit, backward=True)
        return g, None, None


class ParamGate:
    """Residency of the parameter units.  The decoder calls :meth:`enter` before a layer and :meth:`leave` on its
    outputs; everything runs on the current stream, in program order, so a slot is only overwritten after the
    kernels that read its previous contents."""

    def __init__(self, engine: "ShardedParamEngine"):
        self.e = engine
        self.by_layer: dict[tuple[int, int], list[int]] = {}      # (id(layer list owner) , layer) -> bucket indices

    def acquire(self, bucket_index: int, backward: bool = False) -> None:
        """Makes a unit resident for the kernels queued next on the current stream, then starts pulling the unit the
        pass needs after it (the next layer of the same tower going forward, the previous one going backward) on the
        engine's side stream, into the other slot of the pool, so that the pull runs under this layer's kernels."""
        e = self.e
        e._wait_prefetched(bucket_index)
        e._gather_bucket(bucket_index)
        e._prefetch_neighbour(bucket_index, -1 if backward else 1)

    def enter(self, layers: list[nn.Module]) -> list[int]:
        """Makes the units of the given layer modules resident; returns their bucket indices."""
        idx = []
        for layer in layers:
            b = self.e.bucket_of_module(layer)
            if b is not None:
                self.acquire(b)
                idx.append(b)
        return idx

    def leave(self, xs: list[Tensor | None], units: list[int]) -> list[Tensor | None]:
        if not units or not torch.is_grad_enabled():
            return xs
        out = []
        for x in xs:
            if x is not None and x.requires_grad:
                for u in units:
                    x = _BackwardAcquire.apply(x, self, u)
            out.append(x)
        return out


class ShardedParamEngine(TrainEngine):
    """``TrainEngine`` with the parameters themselves sharded (see the module docstring)."""

    _slice_per_bucket = True

    def __init__(self, policy: nn.Module, hyper: OptimHyper, *, device, strategy: str = "fsdp", **kw):
        kw.setdefault("bucket_elems", None)
        self._requested = strategy
        super().__init__(policy, hyper, device=device, strategy="zero2", **kw)

    # the base constructor calls this right after the flat store exists and rank 0's weights have been broadcast
    def _make_store(self, policy, allocator, bucket_elems):
        return FlatParamStore(policy, self.device, pad_to=self.world, allocator=allocator, bucket_key=unit_key)

    def _after_setup(self) -> None:
        self.strategy = "fsdp"
        store, W, r = self.store, self.world, self.rank
        dev = self.device
        self.pshard: list[Tensor] = []
        self._module_bucket: dict[int, int] = {}
        self._slot_of: dict[int, tuple[int, int]] = {}             # bucket -> (group, slot id)
        self._slots: list[list[Tensor]] = []
        self._holds: list[list[int]] = []
        self._gathers = 0
        self._pool_pos: dict[int, tuple[list[int], int]] = {}     # bucket -> (its pool's members in layer order, index)
        self._pending: dict[int, "torch.cuda.Event"] = {}           # bucket -> its prefetch has been queued
        self._prefetch_stream = (torch.cuda.Stream(device=dev) if dev.type == "cuda" and W > 1 and self.p2p is not None
                                 else None)
        for gi, (g, sh) in enumerate(zip(store.groups, self.shards)):
            # at rest: this rank's slices of every bucket, back to back (same order / offsets as the fp32 shard)
            alloc = self.p2p.alloc_symmetric if self.p2p is not None else (
                lambda n, dt: torch.empty(n, dtype=dt, device=dev))
            ps = alloc(sh.numel, g.dtype)
            for (lo, hi), off in zip(sh.slices, sh.offsets):
                ps[off:off + hi - lo].copy_(g.data[lo:hi])
            self.pshard.append(ps)
            # slots: one per root bucket; two rotating ones per tower, as large as the tower's largest layer
            pools: dict[str, list[int]] = {}
            for b in g.buckets:
                key = store.bucket_keys[b.index]
                pools.setdefault("root:" + str(b.index) if key == "root" else key.rsplit("#", 1)[0], []).append(b.index)
            slots, holds = [], []
            for pool, members in pools.items():
                size = max(store.buckets[i].numel for i in members)
                n_slots = 1 if pool.startswith("root:") else min(2, len(members))
                base = len(slots)
                for _ in range(n_slots):
                    slots.append(torch.empty(size, dtype=g.dtype, device=dev))
                    holds.append(-1)
                for j, i in enumerate(members):
                    self._slot_of[i] = (gi, base + (j % n_slots))
                    if n_slots > 1:
                        self._pool_pos[i] = (members, j)
            self._slots.append(slots)
            self._holds.append(holds)
            # parameters become views of their unit's slot; the replicated flat buffer goes away
            for b in g.buckets:
                slot = slots[self._slot_of[b.index][1]]
                for p, o in zip(g.params[b.first_param:b.last_param], g.offsets[b.first_param:b.last_param]):
                    p.data = slot[o - b.lo:o - b.lo + p.numel()].view(p.shape)
            symm = getattr(g.data, "_symm", None)
            g.data = None
            if symm is not None:
                self.p2p._buffers.remove(symm)
                symm.free(self.pg)
        if self.p2p is not None:
            # the optimizer kernel writes the refreshed slice into the LOCAL shard only
            from .comm import MAX_RANKS
            for B in self.p2p.buckets:
                ps = self.pshard[B["bucket"].group]
                B["param_table"] = (c_void_p * MAX_RANKS)(c_void_p(ps.data_ptr()), *[c_void_p(0)] * (MAX_RANKS - 1))
                B["param_world"], B["param_lo"] = 1, B["off"]
        # module -> bucket of its own parameters (decoder layers)
        owner: dict[int, int] = {}
        bucket_of = store.bucket_of_param()
        for mod in self.policy.modules():
            # a layer's adaptive-norm projections live in the root unit: only the layer's OWN unit counts
            own = {bucket_of[id(p)].index for p in mod.parameters() if id(p) in bucket_of}
            own = {i for i in own if store.bucket_keys[i] != "root"}
            if len(own) == 1:
                owner[id(mod)] = own.pop()
        self._module_bucket = owner
        self.gate = ParamGate(self)
        for mod in self.policy.modules():
            if hasattr(mod, "param_gate"):
                mod.param_gate = self.gate
        if self.world > 1:
            if self.device.type == "cuda":
                torch.cuda.synchronize()
            dist.barrier(group=self.pg)                # every rank's at-rest shard is complete before anyone pulls
        self._gather_resident()

    # -- residency ------------------------------------------------------------------------------------------
    def bucket_of_module(self, mod: nn.Module) -> int | None:
        return self._module_bucket.get(id(mod))

    def _gather_bucket(self, index: int, force: bool = False) -> None:
        gi, si = self._slot_of[index]
        if self._holds[gi][si] == index and not force:
            return
        for other in [o for o in self._pending if o != index and self._slot_of[o] == (gi, si)]:
            # an unconsumed prefetch of another unit into this slot: let it finish before the slot is rewritten
            torch.cuda.current_stream().wait_event(self._pending.pop(other))
        b = self.store.buckets[index]
        sh, ps = self.shards[gi], self.pshard[gi]
        k = self.store.groups[gi].buckets.index(b)
        off, n = sh.offsets[k], sh.slices[k][1] - sh.slices[k][0]
        out = self._slots[gi][si][: b.numel]
        if self.world == 1:
            out.copy_(ps[off:off + n])
        elif self.p2p is not None:
            from ..ops import cuda_ops
            from .cp import _ptr_array
            esz = ps.element_size()
            src = [p + off * esz for p in ps._symm.peer_ptrs]
            rc = self.p2p.lib.otb_comm_allgather_pull(_ptr_array(src), c_int(self.world), c_longlong(n * esz),
                                                      c_void_p(out.data_ptr()), c_int(256),
                                                      c_void_p(self.p2p.status),
                                                      c_void_p(torch.cuda.current_stream().cuda_stream))
            if rc != 0:
                raise RuntimeError(f"parameter gather launch failed ({rc})")
            cuda_ops.launch_count += 1
        else:
            mine = ps[off:off + n]
            if dist.get_backend(self.pg) == "nccl":
                dist.all_gather_into_tensor(out, mine, group=self.pg)
            else:
                parts = [torch.empty_like(mine) for _ in range(self.world)]
                dist.all_gather(parts, mine, group=self.pg)
                out.copy_(torch.cat(parts))
        self._holds[gi][si] = index
        self._gathers += 1

    def _wait_prefetched(self, index: int) -> None:
        ev = self._pending.pop(index, None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    def _prefetch_neighbour(self, index: int, step: int) -> None:
        """Queues the pull of the unit ``step`` layers away in the same pool on the side stream.  Its slot holds the
        unit on the other side of ``index``, whose last readers are already queued on the current stream: the side
        stream waits for them first.  The consumer waits for the recorded event (``_wait_prefetched``)."""
        if self._prefetch_stream is None or index not in self._pool_pos:
            return
        members, j = self._pool_pos[index]
        if not 0 <= j + step < len(members):
            return
        nb = members[j + step]
        gi, si = self._slot_of[nb]
        if self._holds[gi][si] == nb or nb in self._pending:
            return
        side = self._prefetch_stream
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._gather_bucket(nb)
            ev = torch.cuda.Event()
            ev.record(side)
        self._pending[nb] = ev

    def _gather_resident(self) -> None:
        for i, key in enumerate(self.store.bucket_keys):
            if key == "root":
                self._gather_bucket(i, force=True)

    def _invalidate(self) -> None:
        if self._pending:                                  # nothing may still be writing a slot that is re-gathered
            for ev in self._pending.values():
                torch.cuda.current_stream().wait_event(ev)
            self._pending.clear()
        for holds in self._holds:
            for i in range(len(holds)):
                holds[i] = -1

    # -- hooks of the base engine -----------------------------------------------------------------------------
    def _param_out(self, gi: int):
        return self.pshard[gi]

    def _params_refreshed(self) -> None:
        """After the optimizer step every slot is stale; root units are needed by the very next kernels."""
        self._invalidate()
        self._gather_resident()

    def _live_slice(self, gi: int, lo: int, hi: int, off: int) -> Tensor:
        return self.pshard[gi][off:off + hi - lo]

    def param_checksum(self) -> Tensor:
        s = torch.zeros(1, dtype=torch.float64, device=self.device)
        for ps in self.pshard:
            s += ps.double().sum()
        if self.world > 1:
            dist.all_reduce(s, group=self.pg)          # every rank holds a different part of one set of parameters
        return s

    @contextmanager
    def full_params(self, writeback: bool = False):
        """Every parameter materialised at once (checkpoint export, loading a state dict, code that walks the module
        tree): a temporary full-size buffer per group.  Collective: every rank must enter.  ``writeback=True``
        copies this rank's slices of the (possibly modified) full values back into the at-rest shards on exit; the
        fp32 masters then have to be rebuilt or loaded by the caller."""
        saved, fulls = [], []
        for gi, g in enumerate(self.store.groups):
            full = torch.empty(g.numel, dtype=g.dtype, device=self.device)
            for b in g.buckets:
                self._gather_bucket(b.index, force=True)
                full[b.lo:b.hi].copy_(self._slots[gi][self._slot_of[b.index][1]][: b.numel])
            for p, o in zip(g.params, g.offsets):
                saved.append((p, p.data))
                p.data = full[o:o + p.numel()].view(p.shape)
            fulls.append(full)
        try:
            yield
        finally:
            for p, d in saved:
                p.data = d
            if writeback:
                for gi, (sh, full) in enumerate(zip(self.shards, fulls)):
                    for (lo, hi), off in zip(sh.slices, sh.offsets):
                        self.pshard[gi][off:off + hi - lo].copy_(full[lo:hi])
                if self.world > 1:
                    if self.device.type == "cuda":
                        torch.cuda.synchronize()
                    dist.barrier(group=self.pg)        # peers read these shards in the gathers below
            self._invalidate()
            self._gather_resident()


def make_engine(policy: nn.Module, hyper: OptimHyper, *, device, strategy: str = "zero2", **kw) -> TrainEngine:
    """The training engine for ``strategy``: ``ddp`` / ``zero1`` / ``zero2`` keep bf16 parameters replicated,
    ``fsdp`` / ``fsdp2`` / ``zero3`` shard them."""
    if strategy in ("fsdp", "fsdp2", "zero3"):
        return ShardedParamEngine(policy, hyper, device=device, strategy=strategy, **kw)
    return TrainEngine(policy, hyper, device=device, strategy=strategy, **kw)
