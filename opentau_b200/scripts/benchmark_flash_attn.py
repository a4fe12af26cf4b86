"""Attention sweep: latency and peak memory of the block-causal kernel against SDPA with the dense mask, forward and
forward+backward, over sequence lengths at the pi0.7-PaliGemma geometry (head_dim 256, MQA), plus a demonstration of the
length at which the dense-mask path runs out of memory while the fused kernel still completes.

Same tables as the reference tool (``src/opentau/scripts/benchmark_flash_attn.py:329-423``); the kernel under test is the
tcgen05 / TMEM one, whose mask is rebuilt from O(S) block ids, so it never holds a (B, H, S, S) tensor.

    python -m opentau_b200.scripts.benchmark_flash_attn [--seqs 1024 2048 4096 8192] [--batch 4] [--oom-demo]
        [--long-context] [--stacked]

``--long-context`` is the forward sweep to ~100 k tokens (reference ``benchmark_flash_attn.py:329-395``); ``--stacked`` is
the training-shaped comparison, a stack of attention layers run forward + backward with and without activation
checkpointing (reference ``benchmark_flash_attn.py:197-265``).  A dense arm is only run where its score and mask tensors
fit a stated budget; beyond it the row says ``skipped`` with the size it would have needed.  Nothing is driven out of
memory on purpose.
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


def _time_and_peak(fn, iters: int = 5, warmup: int = 2) -> tuple[float, float]:
    """``(ms per call, peak GiB above what was held before)`` with CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters, (torch.cuda.max_memory_allocated() - base) / 2**30


def _prefix_lm_blocks(batch: int, s: int, dev):
    from .. import ops
    att = torch.zeros(batch, s, dtype=torch.bool, device=dev)
    att[:, s // 2:] = True
    return ops.make_block_ids(torch.ones(batch, s, dtype=torch.bool, device=dev), att)


def _sdpa_dense(q, k, v, mask, scale):
    g = q.shape[2] // k.shape[2]
    return torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2).repeat_interleave(g, 1), v.transpose(1, 2).repeat_interleave(g, 1),
        attn_mask=mask[:, None], scale=scale).transpose(1, 2)


def long_context_sweep(batch: int = 1, heads: int = 8, kv_heads: int = 1, dim: int = 256,
                       seqs=(4096, 8192, 16384, 32768, 65536, 98304), dense_budget_gib: float = 24.0) -> list[dict]:
    """Forward latency and peak memory against sequence length, prefix-LM mask, bf16.  The fused kernel's mask is
    O(S) block ids; the dense-mask arm needs the (B, S, S) mask plus whatever the library materialises, so it is run
    only while the mask AND a (B, H, S, S) bf16 score tensor fit ``dense_budget_gib``."""
    from .. import ops
    from ..ops import attention_native, cuda_ops
    dev, scale, rows = torch.device("cuda"), dim ** -0.5, []
    for s in seqs:
        q = torch.randn(batch, s, heads, dim, device=dev).to(torch.bfloat16)
        k = torch.randn(batch, s, kv_heads, dim, device=dev).to(torch.bfloat16)
        v = torch.randn(batch, s, kv_heads, dim, device=dev).to(torch.bfloat16)
        blk, valid = _prefix_lm_blocks(batch, s, dev)
        ms, gib = _time_and_peak(lambda: attention_native.attn_fwd(q, k, v, blk, blk, valid, valid, scale))
        cuda_ops.check_status()
        half = s // 2            # prefix rows see the prefix; tail rows see the prefix and the tail up to themselves
        visible = batch * heads * ((s - half) * (s - half) + half * (s - half) + half * (half + 1) / 2)
        rec = {"seq": s, "fused_ms": round(ms, 3), "fused_peak_gib": round(gib, 3),
               "dense_mask_gib": round(batch * s * s / 2**30, 2),
               "fused_tflops_visible": round(4.0 * visible * dim / ms / 1e9, 1)}
        need = (batch * s * s + 2 * batch * heads * s * s) / 2**30
        if need <= dense_budget_gib:
            mask = ops.dense_mask_from_blocks(blk, blk, valid, valid)
            ms_d, gib_d = _time_and_peak(lambda: _sdpa_dense(q, k, v, mask, scale))
            rec.update(sdpa_dense_ms=round(ms_d, 3), sdpa_dense_peak_gib=round(gib_d + batch * s * s / 2**30, 3),
                       vs_sdpa=round(ms_d / ms, 2))
            del mask
        else:
            rec["sdpa_dense"] = f"skipped: mask + scores need ~{need:.0f} GiB (budget {dense_budget_gib:g})"
        rows.append(rec)
        print(json.dumps(rec))
        del q, k, v
        torch.cuda.empty_cache()
    return rows


def stacked_memory_comparison(batch: int = 2, s: int = 1024, heads: int = 8, kv_heads: int = 1, dim: int = 256,
                              layers: int = 18) -> list[dict]:
    """A stack of ``layers`` attention calls (each feeding the next through its output), forward + backward, with and
    without activation checkpointing, for the fused kernel and for SDPA with the dense mask.  Training with
    checkpointing already frees a dense path's per-layer scores by recomputing them, so the ``+ckpt`` rows are the
    like-for-like comparison for training."""
    import torch.utils.checkpoint as cp

    from .. import ops
    dev, scale = torch.device("cuda"), dim ** -0.5
    blk, valid = _prefix_lm_blocks(batch, s, dev)
    mask = ops.dense_mask_from_blocks(blk, blk, valid, valid)
    k = torch.randn(batch, s, kv_heads, dim, device=dev).to(torch.bfloat16)
    v = torch.randn(batch, s, kv_heads, dim, device=dev).to(torch.bfloat16)
    x0 = torch.randn(batch, s, heads, dim, device=dev).to(torch.bfloat16)

    def fused(q):
        return ops.block_attention(q, k, v, blk, blk, valid, valid, scale).reshape(q.shape)   # (B, S, H*D) -> q's

    def dense(q):
        return _sdpa_dense(q, k, v, mask, scale).reshape(q.shape)

    def run(layer, ckpt):
        q = x0.clone().requires_grad_(True)
        h = q
        for _ in range(layers):
            h = cp.checkpoint(layer, h, use_reentrant=False) if ckpt else layer(h)
        h.float().square().mean().backward()

    rows = []
    for name, layer in (("fused", fused), ("sdpa_dense_mask", dense)):
        for ckpt in (False, True):
            ms, gib = _time_and_peak(lambda: run(layer, ckpt), iters=3, warmup=1)
            rec = {"backend": name + ("+ckpt" if ckpt else ""), "layers": layers, "B": batch, "S": s,
                   "fwd_bwd_ms": round(ms, 2), "peak_gib": round(gib, 3)}
            rows.append(rec)
            print(json.dumps(rec))
    return rows


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
    ap.add_argument("--long-context", action="store_true", help="forward sweep to ~100 k tokens at batch 1")
    ap.add_argument("--long-seqs", type=int, nargs="*", default=[4096, 8192, 16384, 32768, 65536, 98304])
    ap.add_argument("--stacked", action="store_true", help="a stack of layers, forward + backward, with / without "
                    "activation checkpointing")
    ap.add_argument("--layers", type=int, default=18)
    ap.add_argument("--stacked-seqs", type=int, nargs="*", default=[1024])
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("this benchmark needs a CUDA device")
    rows = sweep(a.seqs, a.batch, a.heads, a.kv_heads, a.dim, a.iters, a.pattern) if a.seqs else []
    if a.long_context:
        rows += long_context_sweep(1, a.heads, a.kv_heads, a.dim, tuple(a.long_seqs))
    if a.stacked:
        for s in a.stacked_seqs:
            rows += stacked_memory_comparison(min(a.batch, 2), s, a.heads, a.kv_heads, a.dim, a.layers)
    if a.oom_demo:
        print(json.dumps(oom_demo(a.batch, a.heads, a.kv_heads, a.dim)))
    return rows


if __name__ == "__main__":
    main()
