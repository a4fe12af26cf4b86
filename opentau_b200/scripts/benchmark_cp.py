"""Context-parallel attention forward: fused (K/V exchange inside the kernel) against the library baseline
(``all_gather`` of K and V, then the single-GPU kernel), one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29544 \
        -m opentau_b200.scripts.benchmark_cp --batch 2 --seq 12800 --heads 8 --kv-heads 4 --dim 256

Times with CUDA events after warm-up, MAX over ranks; the roofline is the slower of (FLOPs / measured GEMM peak) and
(remote K/V bytes / 770 GB/s).  FLOPs count the visible (unmasked) part of the score matrix only.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .benchmark_kernels import peaks
from .benchmark_tp import NVLINK_GBS, _time


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=12800, help="global sequence length (all ranks together)")
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--dim", type=int, default=256)
    ap.add_argument("--block", type=int, default=256, help="tokens per attention block (frame) of the mask")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--copiers", type=int, default=0, help="copier CTAs of the fused kernel (0: sized from the shape)")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from opentau_b200.ops import cuda_ops, prims
    from opentau_b200.parallel.cp import ContextParallel
    cp = ContextParallel(dev, backend="p2p", num_copiers=a.copiers or None)
    B, S, H, Hkv, D = a.batch, a.seq, a.heads, a.kv_heads, a.dim
    Sl = S // world
    torch.manual_seed(rank)
    q = torch.randn(B, Sl, H, D, device=dev).to(torch.bfloat16)
    k = torch.randn(B, Sl, Hkv, D, device=dev).to(torch.bfloat16)
    v = torch.randn(B, Sl, Hkv, D, device=dev).to(torch.bfloat16)
    blk_all = (torch.arange(S, device=dev, dtype=torch.int32) // a.block)[None].expand(B, S).contiguous()
    ok_all = torch.ones(B, S, dtype=torch.bool, device=dev)
    q_blk, q_ok = cp.shard(blk_all).contiguous(), cp.shard(ok_all).contiguous()
    scale = D ** -0.5
    kf, vf = torch.empty(B, S, Hkv, D, device=dev, dtype=torch.bfloat16), torch.empty(B, S, Hkv, D, device=dev, dtype=torch.bfloat16)

    def fused():
        return cp.attention_forward(q, k, v, q_blk, blk_all, q_ok, ok_all, scale)[0]

    def lib():
        ks, vs = [t.contiguous() for t in kf.chunk(world, 1)], [t.contiguous() for t in vf.chunk(world, 1)]
        dist.all_gather(ks, k)
        dist.all_gather(vs, v)
        return prims.attn_fwd(q, torch.cat(ks, 1), torch.cat(vs, 1), q_blk, blk_all, q_ok, ok_all, scale)[0]

    o1, o2 = fused(), lib()
    torch.cuda.synchronize()
    err = float((o1.float() - o2.float()).abs().max())
    t_f, t_l = _time(fused, a.iters, a.warmup), _time(lib, a.iters, a.warmup)
    cuda_ops.check_status()
    vis = (blk_all[0][None, :] <= q_blk[0][:, None]).float().mean().item()      # visible fraction for this rank's queries
    flops = 4.0 * B * H * Sl * S * D * vis
    link = (world - 1) * 2 * B * Sl * Hkv * D * 2
    pk = peaks()
    roof = max(flops / (pk["tflops"] * 1e9), link / (NVLINK_GBS * 1e6))
    worst = torch.tensor([flops / t_f / 1e9], device=dev)
    dist.all_reduce(worst, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"case": "context-parallel attention fwd", "world": world, "B": B, "S": S, "H": H, "Hkv": Hkv,
                          "D": D, "fused_ms": round(t_f, 4), "library_ms": round(t_l, 4), "speedup": round(t_l / t_f, 3),
                          "rank0_visible_fraction": round(vis, 3), "rank0_tflops": round(flops / t_f / 1e9, 1),
                          "rank0_roofline_ms": round(roof, 4), "rank0_fraction_of_roofline": round(roof / t_f, 3),
                          "peaks": pk["source"], "max_abs_diff_vs_library": round(err, 4)}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
