"""Peer-memory data-parallel step kernels on ONE GPU: the ranks are separate buffers on the same device and each
emulated rank's kernel runs alone (no kernel waits for another launch), so the numbers are the kernels' HBM behaviour
without the link: ``reduce_scatter_kernel`` (sum of W gradient slices -> fp32 shard + squared-norm partials) and
``adamw_allgather_kernel`` (AdamW on the fp32 shard, refreshed parameters stored into every rank's buffer).

    python -m opentau_b200.scripts.benchmark_comm --world 8 --mparams 512 --iters 10

Prints one JSON line per kernel: ms, bytes moved per launch (reads + writes), GB/s and the fraction of the measured
copy bandwidth.  The working set (W gradient buffers, W parameter buffers, four fp32 shard arrays) is far larger than
the 126 MB L2.  The multi-GPU figures of the same kernels are in ``bench.py`` runs (max over ranks).
"""

from __future__ import annotations

import argparse
import json
from ctypes import c_float, c_int, c_longlong, c_void_p
from pathlib import Path

import torch

MAXR = 8


def _table(tensors):
    ptrs = [c_void_p(t.data_ptr()) for t in tensors] + [c_void_p(0)] * (MAXR - len(tensors))
    return (c_void_p * MAXR)(*ptrs)


def _hbm_gbs() -> tuple[float, str]:
    f = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except (KeyError, ValueError):
            pass
    return 6650.0, "fallback"


def main(argv: list[str] | None = None) -> list[dict]:
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--mparams", type=int, default=512, help="parameters of the whole bucket set, in Mi elements")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--blocks", type=int, default=592)
    a = ap.parse_args(argv)
    from ..ops import _lib, cuda_ops
    lib = _lib.load("comm_p2p")
    dev = torch.device("cuda:0")
    W, n = a.world, a.mparams << 20
    shard = n // W
    status = c_void_p(cuda_ops.status_pointer())
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    g = [torch.randn(n, device=dev, dtype=torch.bfloat16) for _ in range(W)]
    p16 = [torch.zeros(n, device=dev, dtype=torch.bfloat16) for _ in range(W)]
    master, m, v = (torch.randn(shard, device=dev), torch.zeros(shard, device=dev), torch.zeros(shard, device=dev))
    g32 = torch.empty(shard, device=dev)
    partial = torch.zeros(max(512, a.blocks), device=dev)
    scale = torch.ones(2, device=dev)
    peak, src = _hbm_gbs()

    def rs(r: int) -> None:
        rc = lib.otb_comm_reduce_scatter(_table(g), c_int(W), c_longlong(r * shard), c_longlong(shard),
                                         c_void_p(g32.data_ptr()), c_void_p(partial.data_ptr()), c_int(a.blocks), c_int(2),
                                         status, stream)
        assert rc == 0, rc

    def ag(r: int) -> None:
        rc = lib.otb_comm_adamw_allgather(
            c_void_p(master.data_ptr()), c_void_p(g32.data_ptr()), c_void_p(m.data_ptr()), c_void_p(v.data_ptr()),
            _table(p16), c_int(W), c_longlong(r * shard), c_longlong(shard), c_float(1e-4), c_float(0.9), c_float(0.95),
            c_float(1e-8), c_float(0.01), c_float(0.1), c_float(0.05), c_void_p(scale.data_ptr()), c_int(a.blocks),
            c_int(2), status, stream)
        assert rc == 0, rc

    out = []
    for name, fn, nbytes in (("reduce_scatter_kernel", rs, shard * (2 * W + 4)),
                             ("adamw_allgather_kernel", ag, shard * (4 * 4 + 3 * 4 + 2 * W))):
        for r in range(3):
            fn(r % W)                                          # warm-up; every call takes another rank's slice
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(a.iters):
            fn(i % W)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / a.iters
        gbs = nbytes / ms / 1e6
        row = {"kernel": name, "world": W, "shard_elems": shard, "ms": round(ms, 4), "bytes_per_launch": nbytes,
               "GBs": round(gbs, 1), f"frac_of_{src}_hbm": round(gbs / peak, 3)}
        print(json.dumps(row))
        out.append(row)
    cuda_ops.check_status()
    return out


if __name__ == "__main__":
    main()
