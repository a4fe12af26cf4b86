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
N_SLOTS = 4
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


class PeerComm:
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
        self.groups: list[dict] = []
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
        """Remembers, per flat group, the symmetric tables of the parameter and gradient buffers."""
        from ..ops import cuda_ops
        self.status = cuda_ops.status_pointer()
        for g, sh in zip(store.groups, shards):
            if g.dtype != torch.bfloat16:
                raise NotImplementedError("the peer-memory step handles bf16 parameter groups")
            n = sh.hi - sh.lo
            self.groups.append(dict(
                group=g, shard=sh, params=g.data._symm, grads=g.grad._symm,
                g32=torch.empty(n, dtype=torch.float32, device=self.device),
                partial=torch.zeros(1024, dtype=torch.float32, device=self.device)))
        self.scale = torch.ones(2, dtype=torch.float32, device=self.device)

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

    def fused_step(self, *, lr: float, hyper, step: int) -> torch.Tensor:
        """reduce-scatter -> norm exchange -> AdamW + all-gather, all over peer memory."""
        from ..ops import cuda_ops
        if len(self.groups) != 1:
            raise NotImplementedError("one bf16 flat group expected")
        self.epoch += 1
        G = self.groups[0]
        sh = G["shard"]
        n = sh.hi - sh.lo
        nblocks = 1024
        self.barrier(0)  # every rank's backward has finished writing its gradient buffer
        rc = self.lib.otb_comm_reduce_scatter(G["grads"].table, c_int(self.world), c_longlong(sh.lo), c_longlong(n),
                                              c_void_p(G["g32"].data_ptr()), c_void_p(G["partial"].data_ptr()),
                                              c_int(nblocks), self._stream())
        if rc != 0:
            raise RuntimeError(f"reduce_scatter launch failed ({rc})")
        rc = self.lib.otb_comm_norm_exchange(
            c_void_p(G["partial"].data_ptr()), c_int(nblocks), self.norms.table, self.flags.table, c_int(self.rank),
            c_int(self.world), c_int(1), c_int(self.epoch), c_float(1.0 / self.world),
            c_float(hyper.grad_clip_norm or 0.0), c_void_p(self.scale.data_ptr()), c_longlong(self.wait_budget),
            c_void_p(self.status), self._stream())
        if rc != 0:
            raise RuntimeError(f"norm_exchange launch failed ({rc})")
        rc = self.lib.otb_comm_adamw_allgather(
            c_void_p(sh.master.data_ptr()), c_void_p(G["g32"].data_ptr()), c_void_p(sh.m.data_ptr()),
            c_void_p(sh.v.data_ptr()), G["params"].table, c_int(self.world), c_longlong(sh.lo), c_longlong(n),
            c_float(lr), c_float(hyper.betas[0]), c_float(hyper.betas[1]), c_float(hyper.eps),
            c_float(hyper.weight_decay), c_float(1.0 - hyper.betas[0] ** step), c_float(1.0 - hyper.betas[1] ** step),
            c_void_p(self.scale.data_ptr()), c_int(nblocks), self._stream())
        if rc != 0:
            raise RuntimeError(f"adamw_allgather launch failed ({rc})")
        cuda_ops.launch_count += 3
        self.barrier(2)  # all ranks' parameter stores have landed; gradients may be cleared
        return self.scale[1].clone()
