"""Attention sweep: latency and peak memory of the block-causal kernel against SDPA with the dense mask, forward and
forward+backward, over sequence lengths at the pi0.7-PaliGemma geometry (head_dim 256, MQA), plus a demonstration of the
length at which the dense-mask path runs out of memory while the fused kernel still completes.

Same tables as the reference tool (``src/opentau/scripts/benchmark_flash_attn.py:329-423``); the kernel under test is the
tcgen05 / TMEM one, whose mask is rebuilt from O(S) block ids, so it never holds a (B, H, S, S) tensor.

    python -m opentau_b200.scripts.benchmark_flash_attn [--seqs 1024 2048 4096 8192] [--batch 4] [--oom-demo]
"""

from __future__ import annotations

import argparse
import json

import torch


def peak_mem_mib(fn) -> float:
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    fn()
    torch.cuda.synchronize()
    return (torch.cuda.max_memory_allocated() - base) / 2**20


def sweep(seqs: list[int], batch: int, heads: int, kv_heads: int, dim: int, iters: int, pattern: str) -> list[dict]:
    from .benchmark_kernels import bench_attention
    rows = []
    for s in seqs:
        tail = {"prefixlm": s // 2, "causal": s, "full": 0}[pattern]
        dense_bytes = batch * heads * s * s * 4
        rec = bench_attention(batch, s, heads, kv_heads, dim, causal_tail=tail, iters=iters,
                              with_sdpa=dense_bytes < 40 * 2**30, backward=True)
        rec["pattern"], rec["dense_scores_gib"] = pattern, round(dense_bytes / 2**30, 2)
        rows.append(rec)
        print(json.dumps(rec))
    return rows


def oom_demo(batch: int, heads: int, kv_heads: int, dim: int, limit_gib: float = 60.0) -> dict:
    """Doubles S until the dense (B,H,S,S) fp32 score tensor alone would exceed ``limit_gib`` (it is never allocated:
    the point is the arithmetic), then runs the fused kernel there and reports its real peak memory."""
    from .. import ops
    from ..ops import attention_native
    s = 1024
    while batch * heads * s * s * 4 / 2**30 < limit_gib:
        s *= 2
    dev = torch.device("cuda")
    q = torch.randn(batch, s, heads, dim, device=dev).to(torch.bfloat16)
    k = torch.randn(batch, s, kv_heads, dim, device=dev).to(torch.bfloat16)
    v = torch.randn(batch, s, kv_heads, dim, device=dev).to(torch.bfloat16)
    att = torch.zeros(batch, s, dtype=torch.bool, device=dev)
    att[:, s // 2:] = True
    blk, valid = ops.make_block_ids(torch.ones(batch, s, dtype=torch.bool, device=dev), att)
    mib = peak_mem_mib(lambda: attention_native.attn_fwd(q, k, v, blk, blk, valid, valid, dim ** -0.5))
    return {"seq": s, "dense_scores_gib": round(batch * heads * s * s * 4 / 2**30, 1), "fused_peak_mib": round(mib, 1)}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--seqs", type=int, nargs="*", default=[1024, 2048, 4096, 8192])
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=1)
    ap.add_argument("--dim", type=int, default=256)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--pattern", default="prefixlm", choices=["prefixlm", "causal", "full"])
    ap.add_argument("--oom-demo", action="store_true")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("this benchmark needs a CUDA device")
    rows = sweep(a.seqs, a.batch, a.heads, a.kv_heads, a.dim, a.iters, a.pattern)
    if a.oom_demo:
        print(json.dumps(oom_demo(a.batch, a.heads, a.kv_heads, a.dim)))
    return rows


if __name__ == "__main__":
    main()
