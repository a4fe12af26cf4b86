"""Per-phase training-step profiler (reference ``src/opentau/scripts/profile_step.py:9-627``).

Same phase vocabulary and JSON keys — ``dataload_wait, forward, bwd, unscale_clip, optim_step, zero_grad_sched,
sync_gather, total`` — but every boundary is a CUDA event on the training stream (one synchronize per step, not
eight), and the throughput comes from the MAX over ranks of the mean step time.  The engine fuses gradient
reduction, clipping and the optimizer into one phase, reported under ``optim_step`` (``unscale_clip`` and
``zero_grad_sched`` are the host-side remainders).  Knobs: ``PROFILE_STEPS`` (default 30), ``PROFILE_WARMUP``
(default 5), ``PROFILE_NO_OPTIM=true`` (skip the optimizer), ``PROFILE_STEP_JSON=<path>``.
"""

from __future__ import annotations

import json
import logging
import os
import time

import torch

from ..configs import parser
from ..configs.train import TrainPipelineConfig
from ..datasets.factory import make_dataset_mixture
from ..datasets.utils import cycle
from ..parallel import control
from ..parallel.engine import OptimHyper, TrainEngine, assemble_weighted_loss
from ..policies.factory import make_policy
from ..utils.logging_utils import init_logging
from ..utils.random_utils import set_seed
from .train import init_distributed, to_device

PHASES = ("dataload_wait", "forward", "bwd", "unscale_clip", "optim_step", "zero_grad_sched", "sync_gather", "total")


class _Clock:
    """CUDA events on the current stream, or ``perf_counter`` on CPU."""

    def __init__(self, device: torch.device):
        self.cuda = device.type == "cuda"
        self.marks: list = []

    def mark(self) -> None:
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.marks.append(e)
        else:
            self.marks.append(time.perf_counter())

    def deltas_ms(self) -> list[float]:
        if self.cuda:
            torch.cuda.synchronize()
            return [a.elapsed_time(b) for a, b in zip(self.marks[:-1], self.marks[1:])]
        return [(b - a) * 1e3 for a, b in zip(self.marks[:-1], self.marks[1:])]


@parser.wrap()
def profile(cfg: TrainPipelineConfig) -> dict:
    rank, world, device = init_distributed()
    init_logging(rank)
    cfg.validate()
    if cfg.gradient_accumulation_steps != 1:
        raise ValueError("profile_step supports gradient_accumulation_steps=1 only")
    steps = int(os.environ.get("PROFILE_STEPS", 30))
    warmup = int(os.environ.get("PROFILE_WARMUP", 5))
    no_optim = os.environ.get("PROFILE_NO_OPTIM", "false").lower() == "true"
    if cfg.seed is not None:
        set_seed(cfg.seed, rank)
    res = make_dataset_mixture(cfg)
    train_mix = res[0] if isinstance(res, tuple) else res
    policy = make_policy(cfg.policy, ds_meta=train_mix.meta).to(device)
    if device.type == "cuda":
        policy.to(torch.bfloat16)
    policy.train()
    opt = cfg.optimizer
    engine = TrainEngine(policy, OptimHyper(lr=opt.lr, betas=tuple(opt.betas), eps=opt.eps, weight_decay=opt.weight_decay,
                                            grad_clip_norm=getattr(opt, "grad_clip_norm", 10.0)),
                         device=device, loss_weights=cfg.loss_weighting, strategy=cfg.distributed.strategy,
                         comm=cfg.distributed.comm)
    loader = cycle(train_mix.get_dataloader(cfg.dataloader_batch_size, cfg.num_workers, rank, world, cfg.prefetch_factor))
    sums = {p: 0.0 for p in PHASES}
    if device.type == "cuda":
        torch.cuda.reset_peak_memory_stats()
    for it in range(warmup + steps):
        clk = _Clock(device)
        t_host = time.perf_counter()
        clk.mark()
        batch = to_device(next(loader), device)
        wait_ms = (time.perf_counter() - t_host) * 1e3
        clk.mark()                                  # -> forward
        losses = policy(batch)
        loss = assemble_weighted_loss(losses, cfg.loss_weighting)
        clk.mark()                                  # -> bwd
        loss.backward()
        clk.mark()                                  # -> unscale_clip (host remainder: fold stray autograd grads)
        engine.store.fold_autograd_grads()
        clk.mark()                                  # -> optim_step (reduce + clip + AdamW + gather, fused)
        if not no_optim:
            engine.optimizer_step()
        clk.mark()                                  # -> zero_grad_sched
        if no_optim:
            engine.store.zero_grad()
        clk.mark()                                  # -> sync_gather
        control.gather_scalars({"loss": loss.detach()}, device=device)
        clk.mark()
        d = clk.deltas_ms()
        if it >= warmup:
            d[0] = max(d[0], wait_ms)
            for name, v in zip(PHASES[:-1], d):
                sums[name] += v
            sums["total"] += sum(d)
    mean = {k: v / steps for k, v in sums.items()}
    per_rank = control.gather_scalars({k: torch.tensor(v) for k, v in mean.items()}, device=device)
    worst = {k: float(v.max()) for k, v in per_rank.items()}
    peak_alloc = torch.cuda.max_memory_allocated() / 2**30 if device.type == "cuda" else 0.0
    peak_res = torch.cuda.max_memory_reserved() / 2**30 if device.type == "cuda" else 0.0
    mem = control.gather_scalars({"alloc": torch.tensor(peak_alloc), "reserved": torch.tensor(peak_res)}, device=device)
    gbs = cfg.dataloader_batch_size * world
    out = {"phases_ms_max_over_ranks": worst, "phases_ms_rank0": {k: float(v[0]) for k, v in per_rank.items()},
           "steps_per_s": 1e3 / worst["total"], "global_samples_per_s": gbs * 1e3 / worst["total"],
           "global_batch_size": gbs, "num_processes": world, "measured_steps": steps, "warmup_steps": warmup,
           "peak_alloc_gib_per_rank": [float(x) for x in mem["alloc"]],
           "peak_reserved_gib_per_rank": [float(x) for x in mem["reserved"]], "no_optim": no_optim,
           "timing": "cuda events" if device.type == "cuda" else "perf_counter"}
    if rank == 0:
        for k in PHASES:
            logging.info("%-16s %9.2f ms", k, worst[k])
        logging.info("throughput: %.2f steps/s, %.1f global samples/s", out["steps_per_s"], out["global_samples_per_s"])
        path = os.environ.get("PROFILE_STEP_JSON")
        if path:
            with open(path, "w") as f:
                json.dump(out, f, indent=2)
    return out


if __name__ == "__main__":
    profile()
