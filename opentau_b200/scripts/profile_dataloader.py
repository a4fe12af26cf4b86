"""Loader-only throughput ceiling per rank (reference ``src/opentau/scripts/profile_dataloader.py:97-236``): iterate
the training dataloader without a model and report samples/s, so a data-bound run can be told from a compute-bound
one.  Knobs: ``PROFILE_BATCHES`` (default 50), ``PROFILE_WARMUP_BATCHES`` (default 5)."""

from __future__ import annotations

import logging
import os
import time

import torch

from ..configs import parser
from ..configs.train import TrainPipelineConfig
from ..datasets.factory import make_dataset_mixture
from ..parallel import control
from ..utils.logging_utils import init_logging
from .train import init_distributed


@parser.wrap()
def profile(cfg: TrainPipelineConfig) -> dict:
    rank, world, device = init_distributed()
    init_logging(rank)
    n = int(os.environ.get("PROFILE_BATCHES", 50))
    warm = int(os.environ.get("PROFILE_WARMUP_BATCHES", 5))
    res = make_dataset_mixture(cfg)
    mix = res[0] if isinstance(res, tuple) else res
    it = iter(mix.get_dataloader(cfg.dataloader_batch_size, cfg.num_workers, rank, world, cfg.prefetch_factor))
    for _ in range(warm):
        next(it)
    t0 = time.perf_counter()
    for _ in range(n):
        next(it)
    dt = time.perf_counter() - t0
    mine = cfg.dataloader_batch_size * n / dt
    allr = control.gather_scalars({"sps": torch.tensor(mine), "ms": torch.tensor(dt / n * 1e3)}, device=device)
    out = {"samples_per_s_per_rank": [float(x) for x in allr["sps"]], "samples_per_s_total": float(allr["sps"].sum()),
           "ms_per_batch_max": float(allr["ms"].max()), "batches": n, "num_workers": cfg.num_workers}
    if rank == 0:
        logging.info("dataloader ceiling: %.1f samples/s over %d rank(s); slowest rank %.1f ms/batch",
                     out["samples_per_s_total"], world, out["ms_per_batch_max"])
    return out


if __name__ == "__main__":
    profile()
