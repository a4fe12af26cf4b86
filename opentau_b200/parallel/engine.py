"""Training engine: one process per GPU, flat bf16 parameters, sharded fp32 AdamW state.

Replaces the reference's ``accelerate`` wrappers (DDP / DeepSpeed ZeRO-1/2/3 / FSDP; OpenTau
``src/opentau/scripts/train.py:219-300,728-1006``) with one explicit step:

    forward -> weighted loss -> backward (weight gradients accumulate into the flat gradient buffer)
    -> gradient reduce-scatter over ranks -> global-norm clip coefficient -> fused AdamW on this rank's
    shard of fp32 masters -> all-gather of the refreshed bf16 parameters.

Numerics contract kept from the reference (``optim/master_weights.py:188-297``): bf16 live weights,
fp32 masters for trainable parameters, L2 clip of the (rank-averaged) gradient at ``grad_clip_norm``
with the pre-clip norm reported, decoupled weight decay, masters rounded to bf16 after the update.
The gradient mean is taken in fp32 (the reference's DDP averages in bf16).

``strategy``: ``"ddp"`` keeps full optimizer state on every rank (all-reduce); ``"zero1"`` / ``"zero2"`` shard the
optimizer state (reduce-scatter + all-gather) and keep the bf16 parameters replicated.  ``comm``: ``"p2p"`` runs the
fused peer-memory kernels, ``"nccl"`` the library collectives (baseline).  Under ``p2p`` the optimizer state is always
sharded (``ddp`` then only names the replicated-parameter layout): a full-state step over peer memory would make
every rank write every parameter into every peer.

Sharding is by gradient bucket: every rank owns an equal slice of EVERY bucket (``parallel/flat.py``), so the
reduce-scatter of a bucket spreads over all ranks and all links, and it starts as soon as the bucket's last
weight-gradient product has been issued (under the rest of the backward pass) instead of after ``backward()``
returns.  The reference gets its overlap from the DDP reducer's buckets (``scripts/train.py:234,594-609``).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Callable

import torch
import torch.distributed as dist
from torch import Tensor, nn

from .. import ops
from .flat import FlatGroup, FlatParamStore


@dataclass
class OptimHyper:
    lr: float = 2.5e-5
    betas: tuple[float, float] = (0.9, 0.95)
    eps: float = 1e-8
    weight_decay: float = 1e-10
    grad_clip_norm: float = 10.0


def assemble_weighted_loss(losses: dict[str, Tensor], weights: dict[str, float]) -> Tensor:
    """``sum_k w_k * loss_k`` over (MSE, CE) in that fixed order; zero-weight terms are dropped from
    the graph (reference ``scripts/train.py:166-216``)."""
    total = None
    for key in ("MSE", "CE"):
        w = float(weights.get(key, 1.0))
        if key not in losses or w == 0.0:
            continue
        term = losses[key] * w if w != 1.0 else losses[key]
        total = term if total is None else total + term
    if total is None:
        raise ValueError("every loss term has zero weight")
    return total


class _ShardState:
    """fp32 masters / moments of this rank's part of one flat group: one slice ``[lo, hi)`` per gradient bucket
    (sharded) or the whole group (replicated), stored back to back; ``offsets[i]`` is where slice ``i`` starts."""

    def __init__(self, group: FlatGroup, rank: int, world: int, sharded: bool, per_bucket: bool = False):
        sharded = sharded and (world > 1 or per_bucket)
        if sharded:
            self.slices = [(b.lo + rank * (b.numel // world), b.lo + (rank + 1) * (b.numel // world))
                           for b in group.buckets]
        else:
            self.slices = [(0, group.numel)]
        self.offsets, off = [], 0
        for lo, hi in self.slices:
            self.offsets.append(off)
            off += hi - lo
        self.numel = off
        dev = group.data.device
        self.master = torch.cat([group.data[lo:hi].float() for lo, hi in self.slices])
        self.m = torch.zeros(off, dtype=torch.float32, device=dev)
        self.v = torch.zeros(off, dtype=torch.float32, device=dev)
        self.contiguous = not sharded                      # the part IS the whole group (no staging needed)
        # staging for the library path when the owned slices are not one contiguous range
        self.grad_stage = None if self.contiguous else torch.empty(off, dtype=group.dtype, device=dev)
        self.param_stage = None if self.contiguous else torch.empty(off, dtype=group.dtype, device=dev)

    def slices_tensor(self) -> Tensor:
        return torch.tensor(self.slices, dtype=torch.int64).reshape(-1, 2)


class TrainEngine:
    _slice_per_bucket = False     # the parameter-sharded engine keeps one slice per bucket even on a single rank

    def __init__(self, policy: nn.Module, hyper: OptimHyper, *, device: torch.device | str,
                 lr_lambda: Callable[[int], float] | None = None, loss_weights: dict[str, float] | None = None,
                 strategy: str = "zero2", comm: str = "auto", process_group=None,
                 grad_accum_steps: int = 1, overlap: bool = True, bucket_elems: int | None = None):
        self.policy = policy
        self.hyper = hyper
        self.device = torch.device(device)
        self.lr_lambda = lr_lambda
        self.loss_weights = loss_weights or {"MSE": 1.0, "CE": 1.0}
        self.pg = process_group
        self.world = dist.get_world_size(process_group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(process_group) if self.world > 1 else 0
        if strategy in ("zero1", "deepspeed"):
            strategy = "zero2"          # gradients are reduce-scattered in both; only the optimizer state is sharded
        if strategy in ("fsdp", "zero3", "fsdp2"):
            raise ValueError(
                f"strategy {strategy!r} shards the PARAMETERS; build the engine with parallel.fsdp.make_engine (or "
                "distributed.strategy in the training config), which wires the per-unit gather into the model")
        if strategy not in ("ddp", "zero2"):
            raise ValueError(f"unknown strategy {strategy!r}")
        self.strategy = strategy if (self.world > 1 or self._slice_per_bucket) else "ddp"
        self.grad_accum_steps = grad_accum_steps
        self.p2p = None
        if comm == "auto":
            comm = "p2p" if (self.world > 1 and self.device.type == "cuda") else "nccl"
        allocator = None
        if comm == "p2p" and self.world > 1:
            from .comm import PeerComm
            self.p2p = PeerComm(self.device, process_group)
            allocator = self.p2p.alloc_symmetric
        self.comm = comm
        if self.p2p is not None:
            self.strategy = "zero2"
        self.store = self._make_store(policy, allocator, bucket_elems)
        if self.world > 1:
            self._broadcast_params()
        sharded = self.sharded_state = self.strategy == "zero2"   # optimizer state (and gradients) sharded by bucket
        self.shards: list[_ShardState] = [_ShardState(g, self.rank, self.world, sharded, self._slice_per_bucket)
                                          for g in self.store.groups]
        self.overlap = bool(overlap) and self.p2p is not None
        if self.p2p is not None:
            self.p2p.register(self.store, self.shards)
            self._install_grad_hooks()
        self.step_count = 0
        self._micro = 0
        n_part = 1024
        self._partials = torch.zeros(len(self.store.groups) * n_part, dtype=torch.float32, device=self.device)
        self._n_part = n_part
        self._scale = torch.ones(2, dtype=torch.float32, device=self.device)
        self.last_grad_norm: Tensor | None = None
        self.store.zero_grad()
        self._after_setup()

    # -- extension points of the parameter-sharded engine (parallel/fsdp.py) ---------------------------------
    def _make_store(self, policy, allocator, bucket_elems) -> FlatParamStore:
        from .flat import DEFAULT_BUCKET_ELEMS
        return FlatParamStore(policy, self.device, pad_to=self.world, allocator=allocator,
                              bucket_elems=bucket_elems or DEFAULT_BUCKET_ELEMS)

    def _after_setup(self) -> None:
        pass

    def _param_out(self, gi: int):
        """Where the library step writes this rank's refreshed parameters of group ``gi`` (None: the replicated
        flat buffer / its staging, followed by an all-gather)."""
        return None

    def _params_refreshed(self) -> None:
        pass

    def _live_slice(self, gi: int, lo: int, hi: int, off: int) -> Tensor:
        return self.store.groups[gi].data[lo:hi]

    def param_checksum(self) -> Tensor:
        """Sum of all trainable parameters as one fp64 device scalar (equal on every rank when the replicas are)."""
        s = torch.zeros(1, dtype=torch.float64, device=self.device)
        for g in self.store.groups:
            s += g.data.double().sum()
        return s

    # -------------------------------------------------------------------------------------------
    def _broadcast_params(self) -> None:
        """Rank 0's initial weights win (DDP init broadcast / FSDP sync_module_states)."""
        for g in self.store.groups:
            dist.broadcast(g.data, src=0, group=self.pg)
        for p in self.policy.parameters():
            if not p.requires_grad:
                dist.broadcast(p.data, src=0, group=self.pg)

    # -- gradient-ready tracking (peer-memory path) ----------------------------------------------------
    def _install_grad_hooks(self) -> None:
        """Every route a parameter gradient can take ends in ``_on_grad``: the fused backward passes that write
        into ``main_grad`` call it through ``ops.fused.set_grad_ready_hook``; gradients that autograd delivers in
        ``.grad`` are folded into ``main_grad`` by a post-accumulate hook first.  The first step only counts how
        many deliveries each parameter gets; later steps reduce a bucket when all its deliveries have happened."""
        from ..ops import fused
        self._bucket_of = self.store.bucket_of_param()
        self._expected: dict[int, int] | None = None
        self._counts: dict[int, int] = {}
        self._remaining: dict[int, int] = {}
        self._bucket_open: dict[int, int] = {}
        self._armed = self._step_open = False
        fused.set_grad_ready_hook(self._on_grad)
        for g in self.store.groups:
            for p in g.params:
                p.register_post_accumulate_grad_hook(self._on_autograd_grad)

    def _on_autograd_grad(self, p) -> None:
        if p.grad is not None:
            p.main_grad.add_(p.grad.to(p.main_grad.dtype))
            p.grad = None
        self._on_grad(p)

    def _on_grad(self, p) -> None:
        b = self._bucket_of.get(id(p))
        if b is None:
            return
        if not self._armed:
            self._counts[id(p)] = self._counts.get(id(p), 0) + 1
            return
        left = self._remaining.get(id(p), 0) - 1
        self._remaining[id(p)] = left
        if left < 0:
            if b.index in self.p2p._reduced:
                raise RuntimeError(
                    "a gradient arrived for a bucket that was already reduced: the backward graph changed since the "
                    "first step (build the engine with overlap=False for models whose graph varies)")
            return
        if left == 0:
            self._bucket_open[b.index] -= 1
            if self._bucket_open[b.index] == 0:
                del self._bucket_open[b.index]
                self.p2p.reduce_bucket_async(b.index, last=not self._bucket_open)

    def _arm(self) -> None:
        """Before the backward pass whose gradients get reduced (the last micro-batch of the step)."""
        self.p2p.begin_step()
        self._step_open = True
        self._armed = self.overlap and self._expected is not None
        if self._armed:
            self._remaining = dict(self._expected)
            self._bucket_open = {}
            for pid, n in self._expected.items():
                if n > 0:
                    i = self._bucket_of[pid].index
                    self._bucket_open[i] = self._bucket_open.get(i, 0) + 1
        else:
            self._counts = {}

    def check(self, blocking: bool = True) -> None:
        """Raises if a bounded wait of the peer-memory step gave up (a peer was late or gone): the step wrote
        nothing, parameters are those of the last good step."""
        if self.p2p is not None:
            self.p2p.check(blocking)

    def current_lr(self) -> float:
        mult = self.lr_lambda(self.step_count) if self.lr_lambda is not None else 1.0
        return self.hyper.lr * mult

    # -------------------------------------------------------------------------------------------
    def forward_backward(self, batch: dict[str, Any]) -> dict[str, Tensor]:
        losses = self.policy(batch)
        loss = assemble_weighted_loss(losses, self.loss_weights)
        if self.grad_accum_steps > 1:
            loss = loss / self.grad_accum_steps
        if self.p2p is not None and self._micro == self.grad_accum_steps - 1:
            self._arm()
        loss.backward()
        self._micro += 1
        out = {k: v.detach() for k, v in losses.items() if isinstance(v, Tensor)}
        out["loss"] = loss.detach() * self.grad_accum_steps
        if losses.get("outlier_records"):
            out["outlier_records"] = losses["outlier_records"]     # host-side debug records, logged by the trainer
        return out

    def optimizer_step(self) -> Tensor:
        """Gradient sync + clip + AdamW + parameter refresh.  Returns the pre-clip gradient norm."""
        self.store.fold_autograd_grads()
        self.step_count += 1
        h = self.hyper
        lr = self.hyper.lr * (self.lr_lambda(self.step_count - 1) if self.lr_lambda is not None else 1.0)
        if self.p2p is not None:
            if not self._step_open:
                self.p2p.begin_step()        # optimizer_step() without forward_backward() (tests, tools)
            if not self._armed and self._expected is None and self._counts:
                self._expected = dict(self._counts)      # deliveries per parameter in one backward pass
            self._armed = self._step_open = False
            norm = self.p2p.fused_step(lr=lr, hyper=h, step=self.step_count)
        else:
            norm = self._library_step(lr)
        self._params_refreshed()
        self.last_grad_norm = norm
        self.store.zero_grad()
        self._micro = 0
        return norm

    def _library_step(self, lr: float) -> Tensor:
        h = self.hyper
        world = self.world
        nccl = world > 1 and dist.get_backend(self.pg) == "nccl"
        grads: list[Tensor] = []
        for g, sh in zip(self.store.groups, self.shards):
            if world > 1 and self.sharded_state:
                if nccl:
                    for b, (lo, hi), off in zip(g.buckets, sh.slices, sh.offsets):
                        dist.reduce_scatter_tensor(sh.grad_stage[off:off + hi - lo], g.grad[b.lo:b.hi],
                                                   op=dist.ReduceOp.SUM, group=self.pg)
                else:
                    dist.all_reduce(g.grad, op=dist.ReduceOp.SUM, group=self.pg)
                    for (lo, hi), off in zip(sh.slices, sh.offsets):
                        sh.grad_stage[off:off + hi - lo].copy_(g.grad[lo:hi])
                shard = sh.grad_stage
            else:
                if world > 1:
                    dist.all_reduce(g.grad, op=dist.ReduceOp.SUM, group=self.pg)
                shard = g.grad
            grads.append(shard)
        # global L2 norm of the rank-averaged gradient
        native = self.device.type == "cuda" and not ops.oracle_mode()
        if native:
            from ..ops import cuda_ops
            self._partials.zero_()
            for i, sg in enumerate(grads):
                cuda_ops.sumsq_partials(sg, self._partials[i * self._n_part:(i + 1) * self._n_part])
            total_sq = self._partials.sum()
        else:
            total_sq = sum((sg.float().pow(2).sum() for sg in grads), torch.zeros((), device=self.device))
        if world > 1 and self.sharded_state:
            dist.all_reduce(total_sq, group=self.pg)
        inv_world = 1.0 / world
        norm = total_sq.sqrt() * inv_world
        if h.grad_clip_norm and h.grad_clip_norm > 0:
            coef = torch.clamp(h.grad_clip_norm / (norm + 1e-6), max=1.0)
        else:
            coef = torch.ones((), device=self.device)
        self._scale[0] = coef * inv_world
        self._scale[1] = norm
        for gi, (g, sh, sg) in enumerate(zip(self.store.groups, self.shards, grads)):
            # the refreshed parameters of this rank's part, in the group's dtype
            local_only = self._param_out(gi)
            p_out = local_only if local_only is not None else (g.data if sh.contiguous else sh.param_stage)
            if native:
                from ..ops import cuda_ops
                if g.dtype == torch.bfloat16:
                    cuda_ops.adamw(sh.master, sg, sh.m, sh.v, p_out, lr=lr, beta1=h.betas[0], beta2=h.betas[1],
                                   eps=h.eps, weight_decay=h.weight_decay, step=self.step_count, scale=self._scale)
                else:
                    cuda_ops.adamw(sh.master, sg, sh.m, sh.v, None, lr=lr, beta1=h.betas[0], beta2=h.betas[1],
                                   eps=h.eps, weight_decay=h.weight_decay, step=self.step_count, scale=self._scale)
                    p_out.copy_(sh.master)
            else:
                ops.ref.adamw_flat(sh.master, sg, sh.m, sh.v, p_out, lr=lr, beta1=h.betas[0], beta2=h.betas[1],
                                   eps=h.eps, weight_decay=h.weight_decay, step=self.step_count,
                                   grad_scale=float(self._scale[0]))
            if world > 1 and self.sharded_state and local_only is None:
                for b, (lo, hi), off in zip(g.buckets, sh.slices, sh.offsets):
                    mine = sh.param_stage[off:off + hi - lo]
                    if nccl:
                        dist.all_gather_into_tensor(g.data[b.lo:b.hi], mine, group=self.pg)
                    else:
                        parts = [torch.empty_like(mine) for _ in range(world)]
                        dist.all_gather(parts, mine, group=self.pg)
                        g.data[b.lo:b.hi].copy_(torch.cat(parts))
        return norm

    def train_step(self, batch: dict[str, Any]) -> dict[str, Tensor]:
        """One optimizer step over ``grad_accum_steps`` calls (returns metrics of this micro-batch)."""
        out = self.forward_backward(batch)
        if self._micro >= self.grad_accum_steps:
            out["grad_norm"] = self.optimizer_step()
            out["lr"] = torch.tensor(self.current_lr())
        return out

    # ------------------------------------------------------------------------------------------- state
    def state_dict(self) -> dict[str, Any]:
        sd: dict[str, Any] = {"step": self.step_count, "rank": self.rank, "world": self.world,
                              "strategy": self.strategy}
        for i, sh in enumerate(self.shards):
            sd[f"group{i}.slices"] = sh.slices_tensor()      # [[lo, hi], ...] inside the flat group, in storage order
            sd[f"group{i}.m"], sd[f"group{i}.v"] = sh.m, sh.v
            sd[f"group{i}.master"] = sh.master
        return sd

    def load_state_dict(self, sd: dict[str, Any], rebuild_masters_from_live: bool = False) -> None:
        self.step_count = int(sd["step"])
        for i, sh in enumerate(self.shards):
            saved = sd.get(f"group{i}.slices")
            if saved is None or saved.reshape(-1, 2).tolist() != [list(x) for x in sh.slices]:
                raise ValueError("optimizer shard layout differs (world size or bucket layout changed); use rebuild")
            sh.m.copy_(sd[f"group{i}.m"])
            sh.v.copy_(sd[f"group{i}.v"])
            if rebuild_masters_from_live or f"group{i}.master" not in sd:
                self._master_from_live(i, sh)
            else:
                sh.master.copy_(sd[f"group{i}.master"])

    def _master_from_live(self, gi: int, sh: _ShardState) -> None:
        for (lo, hi), off in zip(sh.slices, sh.offsets):
            sh.master[off:off + hi - lo].copy_(self._live_slice(gi, lo, hi, off).float())

    def rebuild_masters_from_live(self) -> None:
        for gi, sh in enumerate(self.shards):
            self._master_from_live(gi, sh)
