"""Peer-memory communicator: symmetric buffers over CUDA IPC and the fused data-parallel step.

The reference delegates every collective to NCCL through ``accelerate`` (DDP all-reduce, ZeRO / FSDP
reduce-scatter + all-gather; OpenTau ``src/opentau/scripts/train.py:728-737``).  Here the gradient
reduce-scatter, the global-norm exchange, the sharded AdamW and the parameter all-gather are four kernels
of our own that read and write peers' memory directly over NVLink / NVSwitch
(``ops/csrc/comm_p2p.cu``).  ``torch.distributed`` is used only to exchange the IPC handles once.

Control-plane collectives (metrics, object broadcast, barriers between phases on the host) stay on
``torch.distributed`` — see :mod:`opentau_b200.parallel.control`.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch
import torch.distributed as dist

MAX_RANKS = 8
N_SLOTS = 4            # flag slots of a communicator before a parameter store registers its buckets
DEFAULT_WAIT_BUDGET = 20_000_000_000  # cycles (~10 s): a peer that is this late is treated as failed


class _DeviceBuffer:
    """Wraps a raw device pointer so torch can alias it (``__cuda_array_interface__``)."""

    def __init__(self, ptr: int, nbytes: int):
        self.ptr, self.nbytes = ptr, nbytes
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


class SymmetricBuffer:
    """One allocation per rank, all mapped into every rank."""

    def __init__(self, lib, nbytes: int, device: torch.device, group):
        self.lib, self.nbytes = lib, nbytes
        local = c_void_p(0)
        rc = lib.otb_comm_alloc(c_ulonglong(nbytes), ctypes.byref(local))
        if rc != 0:
            raise RuntimeError(f"symmetric allocation of {nbytes} bytes failed ({rc})")
        self.local_ptr = local.value
        handle = (ctypes.c_ubyte * 64)()
        rc = lib.otb_comm_get_handle(c_void_p(self.local_ptr), handle)
        if rc != 0:
            raise RuntimeError(f"cudaIpcGetMemHandle failed ({rc})")
        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        handles: list = [None] * world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.peer_ptrs: list[int] = []
        self._opened: list[int] = []
        for r, h in enumerate(handles):
            if r == rank:
                self.peer_ptrs.append(self.local_ptr)
                continue
            out = c_void_p(0)
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            rc = lib.otb_comm_open_handle(buf, ctypes.byref(out))
            if rc != 0:
                raise RuntimeError(f"cudaIpcOpenMemHandle for rank {r} failed ({rc})")
            self.peer_ptrs.append(out.value)
            self._opened.append(out.value)
        self.table = (c_void_p * MAX_RANKS)(*[c_void_p(p) for p in self.peer_ptrs],
                                            *[c_void_p(0)] * (MAX_RANKS - world))
        self._holder = _DeviceBuffer(self.local_ptr, nbytes)
        self.bytes_tensor = torch.as_tensor(self._holder, device=device)

    def view(self, dtype: torch.dtype, numel: int) -> torch.Tensor:
        return self.bytes_tensor[: numel * torch.empty(0, dtype=dtype).element_size()].view(dtype)

    def free(self, group=None) -> None:
        """Collective: every rank unmaps its peers' allocations, then releases its own.  The caller must have
        dropped every tensor that aliases the buffer."""
        torch.cuda.synchronize()
        dist.barrier(group=group)
        for p in self._opened:
            self.lib.otb_comm_close_handle(c_void_p(p))
        self._opened = []
        dist.barrier(group=group)
        self.bytes_tensor = self._holder = None
        self.lib.otb_comm_free(c_void_p(self.local_ptr))
        self.local_ptr = 0


class PeerComm:
    """Flag protocol (all waits bounded, every flag carries the step's epoch):

    * slot ``b`` (one per gradient bucket): "my gradients of bucket b are complete".  A rank signals it behind the
      last weight-gradient product of the bucket and waits for every peer's signal before it reads their buckets.
    * slot ``NB``: the squared-norm exchange;  slot ``NB + 1``: "my parameter stores have landed and I no longer
      read anybody's gradients" (end of the step).

    A wait that gives up records ``{kernel, slot, peer}`` in the status word.  From then on the data kernels of the
    step write nothing (they test the word first), so a late or dead peer can stall a step but cannot make this
    rank average half-written gradients into its weights; ``check()`` turns the record into an exception.
    """

    OVERLAP_BLOCKS = 48      # CTAs of a reduce-scatter that runs under the backward pass (leaves the SMs to the GEMMs)
    # CTAs of a reduce-scatter / optimizer kernel that runs alone: two 512-thread CTAs are resident per SM, so 4 x 148
    # fills the GPU in exactly two waves (measured: 296, 512 and 592 CTAs within 7 % of each other, 592 never worst)
    FLUSH_BLOCKS = 592
    PARTIALS_PER_BUCKET = 592

    def __init__(self, device: torch.device, group=None, wait_budget: int = DEFAULT_WAIT_BUDGET):
        from ..ops import _lib
        self.lib = _lib.load("comm_p2p")
        self.device = torch.device(device)
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > MAX_RANKS:
            raise ValueError(f"peer communicator supports up to {MAX_RANKS} ranks per node")
        self.wait_budget = wait_budget
        self._buffers: list[SymmetricBuffer] = []
        self.flags = SymmetricBuffer(self.lib, 4 * MAX_RANKS * N_SLOTS, self.device, group)
        self.norms = SymmetricBuffer(self.lib, 4 * MAX_RANKS, self.device, group)
        self.epoch = 0
        self.buckets: list[dict] = []
        self._reduced: set[int] = set()
        self._pending_check = None
        self.side = torch.cuda.Stream(device=self.device)
        dist.barrier(group=group)

    # -- allocation hook for FlatParamStore -----------------------------------------------------------
    def alloc_symmetric(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        buf = SymmetricBuffer(self.lib, nbytes, self.device, self.group)
        self._buffers.append(buf)
        t = buf.view(dtype, numel)
        t._symm = buf  # keep the mapping alive and reachable from the tensor
        return t

    def register(self, store, shards) -> None:
        """Remembers, per gradient bucket, the symmetric tables of its group's parameter and gradient buffers and
        where this rank's slice of it lives inside the local fp32 shard arrays."""
        from ..ops import cuda_ops
        self.status = cuda_ops.status_pointer()
        nb = len(store.buckets)
        if nb + 2 > N_SLOTS:    # one flag slot per bucket + norm exchange + end of step
            self.flags = SymmetricBuffer(self.lib, 4 * MAX_RANKS * (nb + 2), self.device, self.group)
        self.slot_norm, self.slot_end = nb, nb + 1
        ppb = self.PARTIALS_PER_BUCKET
        self.partial = torch.zeros(nb * ppb, dtype=torch.float32, device=self.device)
        for g, sh in zip(store.groups, shards):
            if g.dtype not in (torch.bfloat16, torch.float32):
                raise NotImplementedError(f"peer-memory step: unsupported parameter dtype {g.dtype}")
            sh.g32 = torch.empty(sh.numel, dtype=torch.float32, device=self.device)
            for b, (lo, hi), off in zip(g.buckets, sh.slices, sh.offsets):
                # where the refreshed parameters of this rank's slice go: every rank's flat parameter buffer
                # (replicated parameters); the parameter-sharded engine redirects it to the local at-rest shard
                self.buckets.append(dict(bucket=b, shard=sh, lo=lo, n=hi - lo, off=off,
                                         param_table=g.data._symm.table, param_world=self.world, param_lo=lo,
                                         grads=g.grad._symm, elem=g.data.element_size(),
                                         partial=self.partial[b.index * ppb:(b.index + 1) * ppb]))
        self.buckets.sort(key=lambda d: d["bucket"].index)
        self.scale = torch.ones(2, dtype=torch.float32, device=self.device)
        # the status word as a tensor + a pinned mirror: each step ends with an asynchronous copy into the mirror,
        # so the next step can look at it without synchronising the device
        self._status_dev = torch.as_tensor(_DeviceBuffer(self.status, 16), device=self.device).view(torch.int32)
        self._status_host = torch.zeros(4, dtype=torch.int32).pin_memory()
        dist.barrier(group=self.group)

    def _stream(self) -> c_void_p:
        return c_void_p(torch.cuda.current_stream().cuda_stream)

    def barrier(self, slot: int) -> None:
        from ..ops import cuda_ops
        rc = self.lib.otb_comm_barrier(self.flags.table, c_int(self.rank), c_int(self.world), c_int(slot),
                                       c_int(self.epoch), c_longlong(self.wait_budget), c_void_p(self.status),
                                       self._stream())
        if rc != 0:
            raise RuntimeError(f"peer barrier launch failed ({rc})")
        cuda_ops.launch_count += 1

    # -- step ------------------------------------------------------------------------------------------
    def begin_step(self) -> None:
        """Called before the backward pass whose gradients will be reduced: opens a new epoch."""
        self.epoch += 1
        self._reduced.clear()

    def _reduce_bucket(self, B: dict, nblocks: int) -> None:
        """On the CURRENT stream: wait until every rank has finished bucket ``B``, then sum this rank's slice."""
        from ..ops import cuda_ops
        self.barrier(B["bucket"].index)
        sh = B["shard"]
        n = B["n"]
        nblocks = max(1, min(nblocks, self.PARTIALS_PER_BUCKET, (n // 8 + 511) // 512))
        if nblocks < self.PARTIALS_PER_BUCKET and B.get("nblocks") not in (None, nblocks):
            B["partial"].zero_()         # fewer blocks than the last launch: stale partials must not be counted
        B["nblocks"] = nblocks
        rc = self.lib.otb_comm_reduce_scatter(B["grads"].table, c_int(self.world), c_longlong(B["lo"]), c_longlong(n),
                                              c_void_p(sh.g32.data_ptr() + 4 * B["off"]),
                                              c_void_p(B["partial"].data_ptr()), c_int(nblocks), c_int(B["elem"]),
                                              c_void_p(self.status), self._stream())
        if rc != 0:
            raise RuntimeError(f"reduce_scatter launch failed ({rc})")
        cuda_ops.launch_count += 1
        self._reduced.add(B["bucket"].index)

    def reduce_bucket_async(self, index: int, last: bool = False) -> None:
        """Bucket ``index`` is complete on this rank as of the work already queued on the current stream: reduce
        it on the side stream, under whatever the backward pass launches next.  ``last``: nothing else of the
        backward pass is left to hide it behind, so it gets the whole GPU."""
        if index in self._reduced:
            raise RuntimeError(f"gradient bucket {index} was reduced twice in one step")
        main = torch.cuda.current_stream()
        self.side.wait_stream(main)
        with torch.cuda.stream(self.side):
            self._reduce_bucket(self.buckets[index], self.FLUSH_BLOCKS if last else self.OVERLAP_BLOCKS)

    def fused_step(self, *, lr: float, hyper, step: int) -> torch.Tensor:
        """Reduce what the backward pass has not reduced yet -> norm exchange -> AdamW + all-gather, all over peer
        memory.  Returns the pre-clip norm of the rank-mean gradient (a device scalar)."""
        from ..ops import cuda_ops
        self.check(blocking=False)
        main = torch.cuda.current_stream()
        main.wait_stream(self.side)                      # overlapped reductions are part of this step
        for B in self.buckets:
            if B["bucket"].index not in self._reduced:
                self._reduce_bucket(B, self.FLUSH_BLOCKS)
        rc = self.lib.otb_comm_norm_exchange(
            c_void_p(self.partial.data_ptr()), c_int(self.partial.numel()), self.norms.table, self.flags.table,
            c_int(self.rank), c_int(self.world), c_int(self.slot_norm), c_int(self.epoch), c_float(1.0 / self.world),
            c_float(hyper.grad_clip_norm or 0.0), c_void_p(self.scale.data_ptr()), c_longlong(self.wait_budget),
            c_void_p(self.status), self._stream())
        if rc != 0:
            raise RuntimeError(f"norm_exchange launch failed ({rc})")
        bc1, bc2 = 1.0 - hyper.betas[0] ** step, 1.0 - hyper.betas[1] ** step
        for B in self.buckets:
            sh, off, n = B["shard"], B["off"], B["n"]
            nblocks = max(1, min(self.FLUSH_BLOCKS, (n // 8 + 511) // 512))
            rc = self.lib.otb_comm_adamw_allgather(
                c_void_p(sh.master.data_ptr() + 4 * off), c_void_p(sh.g32.data_ptr() + 4 * off),
                c_void_p(sh.m.data_ptr() + 4 * off), c_void_p(sh.v.data_ptr() + 4 * off), B["param_table"],
                c_int(B["param_world"]), c_longlong(B["param_lo"]), c_longlong(n), c_float(lr),
                c_float(hyper.betas[0]),
                c_float(hyper.betas[1]), c_float(hyper.eps), c_float(hyper.weight_decay), c_float(bc1), c_float(bc2),
                c_void_p(self.scale.data_ptr()), c_int(nblocks), c_int(B["elem"]), c_void_p(self.status),
                self._stream())
            if rc != 0:
                raise RuntimeError(f"adamw_allgather launch failed ({rc})")
        cuda_ops.launch_count += 1 + len(self.buckets)
        self.barrier(self.slot_end)  # all ranks' parameter stores have landed; gradients may be cleared
        self._status_host.copy_(self._status_dev, non_blocking=True)
        self._pending_check = torch.cuda.Event()
        self._pending_check.record(main)
        return self.scale[1].clone()

    def check(self, blocking: bool = True) -> None:
        """Raises if a wait of an earlier step gave up.  ``blocking=False`` looks only when that step has already
        finished on the device (no synchronisation is added to a pipelined loop); the trainer calls the blocking
        form where it synchronises anyway (reading the loss)."""
        from ..ops import cuda_ops
        ev = self._pending_check
        if ev is None:
            return
        if blocking:
            self._pending_check = None
            cuda_ops.check_status()
        elif ev.query():
            self._pending_check = None
            if int(self._status_host[0]) != 0:      # the mirror is complete once the event is: no device sync here
                cuda_ops.check_status()
