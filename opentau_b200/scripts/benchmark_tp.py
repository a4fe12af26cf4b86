"""Fused tensor-parallel linears against their library baselines, one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        -m opentau_b200.scripts.benchmark_tp --tokens 8192 --hidden 5120 --ffn 25600 --heads 64 --kv-heads 8

For the two shapes of a Qwen3-VL-32B-style layer (attention: qkv column-parallel + o row-parallel; MLP: gate/up
column-parallel + down row-parallel) it times, with CUDA events after warm-up and as the MAX over ranks:

* ``fused_ag_gemm``  — the all-gather happens as TMA loads from the owners' memory inside the GEMM kernel
* ``nccl_ag_gemm``   — ``all_gather_into_tensor`` followed by the plain tcgen05 GEMM
* ``fused_gemm_rs``  — partial tiles stored into the destination rank from the GEMM epilogue, reduced in the kernel tail
* ``nccl_gemm_rs``   — plain GEMM followed by ``reduce_scatter_tensor``

and reports each fused path's fraction of its roofline: the slower of (FLOPs / measured GEMM peak) and (bytes that
must cross NVLink / 770 GB/s per direction).  Rank 0 prints one JSON line per case.  The reference has no fused
counterpart (its collectives are NCCL calls issued by accelerate / DeepSpeed).
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .benchmark_kernels import peaks

NVLINK_GBS = 770.0


def _time(fn, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192, help="global rows M (all ranks together)")
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--ffn", type=int, default=25600)
    ap.add_argument("--heads", type=int, default=64)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from opentau_b200.ops import cuda_ops
    from opentau_b200.parallel.tp import TensorParallel
    tp = TensorParallel(dev, backend="p2p")
    pk = peaks()
    M, d = args.tokens, args.hidden
    Ml = M // world
    qkv_n = (args.heads + 2 * max(args.kv_heads, world)) * args.head_dim // world
    cases = [("qkv", "ag", qkv_n, d), ("gate_up", "ag", 2 * args.ffn // world, d),
             ("o_proj", "rs", d, args.heads * args.head_dim // world), ("down", "rs", d, args.ffn // world)]
    torch.manual_seed(rank)
    for name, kind, N, K in cases:
        w = (torch.randn(N, K, device=dev) / K ** 0.5).to(torch.bfloat16)
        flops = 2.0 * M * N * K
        if kind == "ag":
            x_local = torch.randn(Ml, K, device=dev).to(torch.bfloat16)
            gathered = torch.empty(M, K, device=dev, dtype=torch.bfloat16)

            def fused():
                return tp.all_gather_linear(x_local, w)

            def lib():
                dist.all_gather_into_tensor(gathered, x_local)
                return cuda_ops.gemm(gathered, w, "nt")

            link_bytes = (world - 1) * Ml * K * 2          # what one rank must pull in
        else:
            x = torch.randn(M, K, device=dev).to(torch.bfloat16)
            out_l = torch.empty(Ml, N, device=dev, dtype=torch.bfloat16)

            def fused():
                return tp.linear_reduce_scatter(x, w)

            def lib():
                part = cuda_ops.gemm(x, w, "nt")
                dist.reduce_scatter_tensor(out_l, part)
                return out_l

            link_bytes = (world - 1) * Ml * N * 2          # partial tiles one rank must push out
        a, b = fused(), lib()
        torch.cuda.synchronize()
        err = float((a.float() - b.float()).abs().max())
        t_f = _time(fused, args.iters, args.warmup)
        t_l = _time(lib, args.iters, args.warmup)
        cuda_ops.check_status()
        roof_ms = max(flops / (pk["tflops"] * 1e9), link_bytes / (NVLINK_GBS * 1e6))
        if rank == 0:
            print(json.dumps({
                "case": f"{name}:{'all_gather->gemm' if kind == 'ag' else 'gemm->reduce_scatter'}", "world": world,
                "M": M, "N_local" if kind == "ag" else "N": N, "K" if kind == "ag" else "K_local": K,
                "fused_ms": round(t_f, 4), "library_ms": round(t_l, 4), "speedup": round(t_l / t_f, 3),
                "tflops_per_gpu": round(flops / t_f / 1e9, 1), "roofline_ms": round(roof_ms, 4),
                "fraction_of_roofline": round(roof_ms / t_f, 3), "peaks": pk["source"],
                "max_abs_diff_vs_library": round(err, 4)}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
