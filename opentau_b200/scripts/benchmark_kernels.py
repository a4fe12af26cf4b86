"""Kernel micro-benchmarks: tcgen05 GEMM, block-causal attention and the memory-bound kernels.

Counterpart of the reference's attention benchmark (OpenTau ``src/opentau/scripts/benchmark_flash_attn.py``),
extended to every hot kernel.  Times with CUDA events after warm-up, rotates through enough distinct
input buffers to exceed the 126 MB L2 between iterations, and prints one JSON line per case with the
achieved rate and its fraction of the measured peaks (``MEASURED_PEAKS.json`` next to the package when
present, else 1.59 PFLOP/s / 6.65 TB/s).

    python -m opentau_b200.scripts.benchmark_kernels gemm --m 8192 --n 8192 --k 8192 [--layout nt]
    python -m opentau_b200.scripts.benchmark_kernels attention --batch 32 --sq 1227 --heads 8 --kv-heads 1 --dim 256
    python -m opentau_b200.scripts.benchmark_kernels suite
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch


def peaks() -> dict:
    f = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return {"tflops": d["bf16_tflops"], "tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "gbs": d["hbm_gbs"], "source": "measured"}
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "gbs": 6650.0, "source": "fallback"}


def time_ms(fns, iters: int = 20, warmup: int = 3) -> float:
    """Mean time of one call; ``fns`` is a list of closures over distinct buffers used round-robin."""
    for i in range(warmup):
        fns[i % len(fns)]()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fns[i % len(fns)]()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _n_buffers(bytes_per_set: int) -> int:
    return max(1, min(8, (160 << 20) // max(1, bytes_per_set) + 1))


def bench_gemm(M, N, K, layout="nt", iters=20, with_torch=True, glu=None) -> dict:
    from opentau_b200.ops import cuda_ops
    dev = torch.device("cuda")
    shape_a = (M, K) if layout != "tn" else (K, M)
    shape_b = (N, K) if layout == "nt" else (K, N)
    nb = _n_buffers(2 * (M * K + N * K + M * N))
    As = [torch.randn(shape_a, device=dev).to(torch.bfloat16) for _ in range(nb)]
    Bs = [torch.randn(shape_b, device=dev).to(torch.bfloat16) for _ in range(nb)]
    outs = [torch.empty(M, N, device=dev, dtype=torch.bfloat16) for _ in range(nb)]
    if glu:
        h = [torch.empty(M, N // 2, device=dev, dtype=torch.bfloat16) for _ in range(nb)]
        fns = [lambda a=a, b=b, o=o, hh=hh: cuda_ops.gemm(a, b, layout, out=o, glu=glu, glu_out=hh)
               for a, b, o, hh in zip(As, Bs, outs, h)]
    else:
        fns = [lambda a=a, b=b, o=o: cuda_ops.gemm(a, b, layout, out=o) for a, b, o in zip(As, Bs, outs)]
    ms = time_ms(fns, iters)
    cuda_ops.check_status()
    pk = peaks()
    tf = 2.0 * M * N * K / ms / 1e9
    rec = {"kernel": "gemm_tcgen05", "layout": layout, "M": M, "N": N, "K": K, "glu": glu, "ms": round(ms, 4),
           "tflops": round(tf, 1), f"frac_of_{pk['source']}_peak": round(tf / pk["tflops"], 3), "buffers": nb}
    if with_torch:
        if layout == "nt":
            tf_fns = [lambda a=a, b=b, o=o: torch.matmul(a, b.t(), out=o) for a, b, o in zip(As, Bs, outs)]
        elif layout == "nn":
            tf_fns = [lambda a=a, b=b, o=o: torch.matmul(a, b, out=o) for a, b, o in zip(As, Bs, outs)]
        else:
            tf_fns = [lambda a=a, b=b, o=o: torch.matmul(a.t(), b, out=o) for a, b, o in zip(As, Bs, outs)]
        ms_t = time_ms(tf_fns, iters)
        rec["cublas_ms"] = round(ms_t, 4)
        rec["cublas_tflops"] = round(2.0 * M * N * K / ms_t / 1e9, 1)
        rec["vs_cublas"] = round(ms_t / ms, 3)
    return rec


def bench_skinny(shapes: list[tuple[int, int, int]], iters: int = 20) -> list[dict]:
    """Few-row ``x @ W^T`` products (inference): the weight-streaming split-K kernel at every cluster size, the
    persistent 128-row kernel, and the library GEMM; weights rotate through buffers larger than L2."""
    from opentau_b200.ops import cuda_ops
    dev = torch.device("cuda")
    pk = peaks()
    rows = []
    for M, N, K in shapes:
        nb = _n_buffers(2 * N * K)
        xs = [torch.randn(M, K, device=dev).to(torch.bfloat16) for _ in range(nb)]
        ws = [torch.randn(N, K, device=dev).to(torch.bfloat16) for _ in range(nb)]
        rec = {"kernel": "gemm_skinny_tcgen05", "M": M, "N": N, "K": K}
        best = None
        for s_ in (0, 1, 2, 3, 4, 6, 8):
            if s_ and (K + 63) // 64 < 2 * s_:
                continue
            try:
                ms = time_ms([lambda x=x, w=w: cuda_ops.gemm(x, w, "nt", splits=s_ or (0 if cuda_ops.use_skinny(
                    "nt", M, N, False, 0) else 1)) for x, w in zip(xs, ws)], iters)
            except RuntimeError:
                continue
            rec[f"splits{s_ or '_auto'}_us"] = round(ms * 1e3, 2)
            if s_:
                best = ms if best is None else min(best, ms)
        cuda_ops.check_status()
        rec["persistent_us"] = round(time_ms([lambda x=x, w=w: cuda_ops.gemm(x, w, "nt", bn=128 if N < 4096 else 256)
                                              for x, w in zip(xs, ws)], iters) * 1e3, 2)
        rec["library_us"] = round(time_ms([lambda x=x, w=w: x @ w.t() for x, w in zip(xs, ws)], iters) * 1e3, 2)
        stream_gbs = 2 * N * K / (rec["splits_auto_us"] * 1e-6) / 1e9
        rec["weight_stream_gbs_auto"] = round(stream_gbs, 1)
        rec[f"frac_of_{pk['source']}_hbm"] = round(stream_gbs / pk["gbs"], 3)
        rows.append(rec)
        print(json.dumps(rec))
    return rows


def graph_us(fns, reps: int = 10) -> float:
    """Per-call device time of a chain of launches replayed from one CUDA graph (no host launch cost): what a call
    costs inside the captured sampler."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for f in fns:
            f()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fns:
            f()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * len(fns))


def bench_skinny_graph(shapes: list[tuple[int, int, int]], chain: int = 32) -> list[dict]:
    """The few-row products replayed from a CUDA graph, `chain` launches over rotating weights, per cluster size."""
    from opentau_b200.ops import cuda_ops
    dev = torch.device("cuda")
    rows = []
    for M, N, K in shapes:
        nb = max(_n_buffers(2 * N * K), 4)
        xs = [torch.randn(M, K, device=dev).to(torch.bfloat16) for _ in range(nb)]
        ws = [torch.randn(N, K, device=dev).to(torch.bfloat16) for _ in range(nb)]
        outs = [torch.empty(M, N, device=dev, dtype=torch.bfloat16) for _ in range(nb)]
        rec = {"kernel": "gemm_skinny_tcgen05 (graph replay)", "M": M, "N": N, "K": K}
        for s_ in (1, 2, 3, 4, 6, 8):
            if (K + 63) // 64 < 2 * s_:
                continue
            fns = [lambda i=i: cuda_ops.gemm(xs[i % nb], ws[i % nb], "nt", out=outs[i % nb], splits=s_)
                   for i in range(chain)]
            rec[f"splits{s_}_us"] = round(graph_us(fns), 2)
        fns = [lambda i=i: cuda_ops.gemm(xs[i % nb], ws[i % nb], "nt", out=outs[i % nb], bn=128 if N < 4096 else 256)
               for i in range(chain)]
        rec["persistent_us"] = round(graph_us(fns), 2)
        fns = [lambda i=i: torch.matmul(xs[i % nb], ws[i % nb].t(), out=outs[i % nb]) for i in range(chain)]
        rec["library_us"] = round(graph_us(fns), 2)
        rec["hbm_floor_us"] = round(2 * N * K / peaks()["gbs"] / 1e3, 2)
        cuda_ops.check_status()
        rows.append(rec)
        print(json.dumps(rec), flush=True)
    return rows


# (rows, out features, in features): pi0.5 expert / cosmos3 expert, backbone prefix and vision tower products
SKINNY_SHAPES = [(51, 2560, 1024), (51, 1024, 2048), (51, 8192, 1024), (51, 1024, 4096),
                 (51, 4096, 1024), (51, 1024, 2048), (211, 10240, 5120), (211, 5120, 8192), (211, 51200, 5120),
                 (211, 5120, 25600), (588, 3456, 1152), (588, 1152, 1152), (588, 4304, 1152), (588, 1152, 4304),
                 (968, 2560, 2048), (968, 32768, 2048), (968, 2048, 16384)]


def bench_attention(B, Sq, H, Hkv, D, cross=0, causal_tail=0, iters=20, with_sdpa=True, backward=False) -> dict:
    from opentau_b200 import ops
    from opentau_b200.ops import attention_native, cuda_ops
    dev = torch.device("cuda")
    Sk = Sq + cross
    nb = _n_buffers(2 * B * (Sq * H + 2 * Sk * Hkv) * D)
    qs = [torch.randn(B, Sq, H, D, device=dev).to(torch.bfloat16) for _ in range(nb)]
    ks = [torch.randn(B, Sk, Hkv, D, device=dev).to(torch.bfloat16) for _ in range(nb)]
    vs = [torch.randn(B, Sk, Hkv, D, device=dev).to(torch.bfloat16) for _ in range(nb)]
    att = torch.zeros(B, Sq, dtype=torch.bool, device=dev)
    if causal_tail:
        att[:, Sq - causal_tail:] = True
    pad = torch.ones(B, Sq, dtype=torch.bool, device=dev)
    q_blk, q_valid = ops.make_block_ids(pad, att)
    if cross:
        k_blk = torch.cat([torch.full((B, cross), ops.INT_MIN, dtype=torch.int32, device=dev), q_blk], 1)
        k_valid = torch.cat([torch.ones(B, cross, dtype=torch.bool, device=dev), q_valid], 1)
    else:
        k_blk, k_valid = q_blk, q_valid
    scale = D ** -0.5
    mask = ops.dense_mask_from_blocks(q_blk, k_blk, q_valid, k_valid)
    visible = float(mask.sum().item()) * H
    flops = 4.0 * visible * D
    fns = [lambda q=q, k=k, v=v: attention_native.attn_fwd(q, k, v, q_blk, k_blk, q_valid, k_valid, scale)
           for q, k, v in zip(qs, ks, vs)]
    ms = time_ms(fns, iters)
    cuda_ops.check_status()
    pk = peaks()
    rec = {"kernel": "attn_fwd_tcgen05", "B": B, "Sq": Sq, "Sk": Sk, "H": H, "Hkv": Hkv, "D": D, "ms": round(ms, 4),
           "tflops_visible": round(flops / ms / 1e9, 1),
           f"frac_of_{pk['source']}_peak": round(flops / ms / 1e9 / pk["tflops"], 3)}
    if backward and attention_native.supported_bwd(qs[0], ks[0], vs[0]):
        o, lse = attention_native.attn_fwd(qs[0], ks[0], vs[0], q_blk, k_blk, q_valid, k_valid, scale)
        do = torch.randn_like(o)
        bfn = [lambda q=q, k=k, v=v: attention_native.attn_bwd(do, q, k, v, o, lse, q_blk, k_blk, q_valid, k_valid,
                                                               scale) for q, k, v in zip(qs, ks, vs)]
        ms_b = time_ms(bfn, iters)
        cuda_ops.check_status()
        rec["bwd_ms"] = round(ms_b, 4)
        rec["bwd_tflops_visible"] = round(2.5 * flops / ms_b / 1e9, 1)
    if with_sdpa:
        g = H // Hkv
        am = mask[:, None]
        sd = [lambda q=q, k=k, v=v: torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2).repeat_interleave(g, 1), v.transpose(1, 2).repeat_interleave(g, 1),
            attn_mask=am, scale=scale) for q, k, v in zip(qs, ks, vs)]
        ms_s = time_ms(sd, iters)
        rec["sdpa_dense_mask_ms"] = round(ms_s, 4)
        rec["vs_sdpa"] = round(ms_s / ms, 3)
    return rec


def bench_attention_f32(B, Sq, H, Hkv, D, causal_tail=0, iters=10) -> dict:
    """The exact fp32 kernels (``csrc/attention_f32.cu``) against the dense fp32 PyTorch evaluation of the same masked
    attention (which materialises the ``(B, H, Sq, Sk)`` scores), forward and backward, with the peak memory of each."""
    from opentau_b200 import ops
    from opentau_b200.ops import attention as dispatch
    from opentau_b200.ops import attention_native
    dev = torch.device("cuda")
    q = torch.randn(B, Sq, H, D, device=dev)
    k = torch.randn(B, Sq, Hkv, D, device=dev)
    v = torch.randn(B, Sq, Hkv, D, device=dev)
    att = torch.zeros(B, Sq, dtype=torch.bool, device=dev)
    if causal_tail:
        att[:, Sq - causal_tail:] = True
    q_blk, q_valid = ops.make_block_ids(torch.ones(B, Sq, dtype=torch.bool, device=dev), att)
    scale = D ** -0.5
    visible = float(ops.dense_mask_from_blocks(q_blk, q_blk, q_valid, q_valid).sum().item()) * H
    flops = 4.0 * visible * D
    assert attention_native.supported_f32(q, k, v)
    o, lse = attention_native.attn_f32_fwd(q, k, v, q_blk, q_blk, q_valid, q_valid, scale)
    do = torch.randn_like(o)
    rec = {"kernel": "attn_f32", "B": B, "Sq": Sq, "H": H, "Hkv": Hkv, "D": D}

    def timed(fn):
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        ms = time_ms([fn], iters)
        return ms, (torch.cuda.max_memory_allocated() - base) / 2**20

    ms, mem = timed(lambda: attention_native.attn_f32_fwd(q, k, v, q_blk, q_blk, q_valid, q_valid, scale))
    rec.update(fwd_ms=round(ms, 3), fwd_tflops_visible=round(flops / ms / 1e9, 2), fwd_extra_mib=round(mem, 1))
    ms, mem = timed(lambda: attention_native.attn_f32_bwd(do, q, k, v, o, lse, q_blk, q_blk, q_valid, q_valid, scale))
    rec.update(bwd_ms=round(ms, 3), bwd_tflops_visible=round(2.5 * flops / ms / 1e9, 2), bwd_extra_mib=round(mem, 1))
    ms, mem = timed(lambda: dispatch.dense_attn_fwd(q, k, v, q_blk, q_blk, q_valid, q_valid, scale))
    rec.update(dense_fwd_ms=round(ms, 3), dense_fwd_extra_mib=round(mem, 1))
    ms, mem = timed(lambda: dispatch.dense_attn_bwd(do, q, k, v, o, lse, q_blk, q_blk, q_valid, q_valid, scale))
    rec.update(dense_bwd_ms=round(ms, 3), dense_bwd_extra_mib=round(mem, 1))
    rec["fwd_speedup"] = round(rec["dense_fwd_ms"] / rec["fwd_ms"], 2)
    rec["bwd_speedup"] = round(rec["dense_bwd_ms"] / rec["bwd_ms"], 2)
    return rec


def bench_stss(B=32, T=4, HW=16, C=256, L=5, k=9, iters=10) -> dict:
    """Space-time window correlation: the kernels (``csrc/stss_corr.cu``) against the unfold + einsum evaluation, forward
    and forward + backward, with the extra memory each needs."""
    from opentau_b200.ops import stss
    dev = torch.device("cuda")
    x = torch.nn.functional.normalize(torch.randn(B, T, HW * HW, C, device=dev), dim=-1).to(torch.bfloat16)
    rec = {"kernel": "stss_corr", "B": B, "T": T, "grid": HW, "C": C, "L": L, "k": k}

    def run(fn, backward):
        def step():
            xr = x.detach().requires_grad_(backward)
            out = fn(xr, T, HW, HW, L, k)
            if backward:
                out.backward(torch.ones_like(out))
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        ms = time_ms([step], iters)
        return round(ms, 3), round((torch.cuda.max_memory_allocated() - base) / 2**20, 1)

    rec["fwd_ms"], rec["fwd_extra_mib"] = run(stss.local_window_correlation, False)
    rec["fwd_bwd_ms"], rec["fwd_bwd_extra_mib"] = run(stss.local_window_correlation, True)
    rec["dense_fwd_ms"], rec["dense_fwd_extra_mib"] = run(stss.dense_window_correlation, False)
    rec["dense_fwd_bwd_ms"], rec["dense_fwd_bwd_extra_mib"] = run(stss.dense_window_correlation, True)
    rec["fwd_speedup"] = round(rec["dense_fwd_ms"] / rec["fwd_ms"], 2)
    rec["fwd_bwd_speedup"] = round(rec["dense_fwd_bwd_ms"] / rec["fwd_bwd_ms"], 2)
    return rec


def bench_membound(rows=39264, H=2048, iters=20) -> list[dict]:
    from opentau_b200.ops import cuda_ops
    dev = torch.device("cuda")
    pk = peaks()
    out = []
    nb = _n_buffers(4 * rows * H)
    xs = [torch.randn(rows, H, device=dev).to(torch.bfloat16) for _ in range(nb)]
    w = torch.randn(H, device=dev).to(torch.bfloat16)
    ms = time_ms([lambda x=x: cuda_ops.rms_fwd(x, w, 1e-6, True) for x in xs], iters)
    gb = 2 * rows * H * 2 / 1e9
    out.append({"kernel": "rms_fwd", "rows": rows, "H": H, "ms": round(ms, 4), "GBs": round(gb / ms * 1e3, 1),
                f"frac_of_{pk['source']}_hbm": round(gb / ms * 1e3 / pk["gbs"], 3)})
    I = 4 * H
    gus = [torch.randn(rows // 4, 2 * I, device=dev).to(torch.bfloat16) for _ in range(nb)]
    ms = time_ms([lambda g=g: cuda_ops.glu_fwd(g, "gelu_tanh") for g in gus], iters)
    gb = (rows // 4) * 3 * I * 2 / 1e9
    out.append({"kernel": "glu_fwd", "rows": rows // 4, "I": I, "ms": round(ms, 4), "GBs": round(gb / ms * 1e3, 1),
                f"frac_of_{pk['source']}_hbm": round(gb / ms * 1e3 / pk["gbs"], 3)})
    n = 256 << 20
    p32, m, v = (torch.zeros(n, device=dev) for _ in range(3))
    g = torch.randn(n, device=dev).to(torch.bfloat16)
    p16 = torch.empty(n, device=dev, dtype=torch.bfloat16)
    ms = time_ms([lambda: cuda_ops.adamw(p32, g, m, v, p16, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8,
                                         weight_decay=0.0, step=1)], 10)
    gb = n * (3 * 4 * 2 + 2 + 2) / 1e9
    out.append({"kernel": "adamw", "n": n, "ms": round(ms, 4), "GBs": round(gb / ms * 1e3, 1),
                f"frac_of_{pk['source']}_hbm": round(gb / ms * 1e3 / pk["gbs"], 3)})
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8192)
    g.add_argument("--n", type=int, default=8192)
    g.add_argument("--k", type=int, default=8192)
    g.add_argument("--layout", default="nt")
    g.add_argument("--iters", type=int, default=20)
    g.add_argument("--glu", default=None)
    g.add_argument("--no-torch", action="store_true")
    a = sub.add_parser("attention")
    a.add_argument("--batch", type=int, default=32)
    a.add_argument("--sq", type=int, default=1227)
    a.add_argument("--heads", type=int, default=8)
    a.add_argument("--kv-heads", type=int, default=1)
    a.add_argument("--dim", type=int, default=256)
    a.add_argument("--cross", type=int, default=0)
    a.add_argument("--causal-tail", type=int, default=259)
    a.add_argument("--iters", type=int, default=20)
    a.add_argument("--no-sdpa", action="store_true")
    a.add_argument("--backward", action="store_true")
    a.add_argument("--fp32", action="store_true", help="the exact fp32 kernels against the dense fp32 evaluation")
    sub.add_parser("membound")
    sub.add_parser("stss")
    sk = sub.add_parser("skinny")
    sk.add_argument("--shape", type=int, nargs=3, action="append", default=None, metavar=("M", "N", "K"))
    sk.add_argument("--iters", type=int, default=20)
    sk.add_argument("--graph", action="store_true", help="time the launches inside a replayed CUDA graph")
    sub.add_parser("suite")
    args = ap.parse_args(argv)
    if args.cmd == "gemm":
        print(json.dumps(bench_gemm(args.m, args.n, args.k, args.layout, args.iters, not args.no_torch, args.glu)))
    elif args.cmd == "attention" and args.fp32:
        print(json.dumps(bench_attention_f32(args.batch, args.sq, args.heads, args.kv_heads, args.dim, args.causal_tail,
                                             args.iters)))
    elif args.cmd == "attention":
        print(json.dumps(bench_attention(args.batch, args.sq, args.heads, args.kv_heads, args.dim, args.cross,
                                         args.causal_tail, args.iters, not args.no_sdpa, args.backward)))
    elif args.cmd == "stss":
        print(json.dumps(bench_stss()))
    elif args.cmd == "membound":
        for r in bench_membound():
            print(json.dumps(r))
    elif args.cmd == "skinny":
        shapes = [tuple(x) for x in args.shape] if args.shape else SKINNY_SHAPES
        bench_skinny_graph(shapes) if args.graph else bench_skinny(shapes, args.iters)
    else:
        M = 39264
        for (l, m, n, k, glu) in [("nt", 8192, 8192, 8192, None), ("nt", M, 2560, 2048, None),
                                  ("nt", M, 32768, 2048, "gelu_tanh"), ("nt", M, 2048, 16384, None),
                                  ("nn", M, 2048, 32768, None), ("tn", 32768, 2048, M, None),
                                  ("nn", M, 16384, 2048, None), ("tn", 2048, 16384, M, None),
                                  ("nt", 24576, 3456, 1152, None), ("nt", 24576, 4304, 1152, None),
                                  ("nt", 1600, 2560, 1024, None), ("nt", 1600, 8192, 1024, None)]:
            print(json.dumps(bench_gemm(m, n, k, l, glu=glu)), flush=True)
        for kw in [dict(B=32, Sq=1227, H=8, Hkv=1, D=256, causal_tail=259),
                   dict(B=32, Sq=50, H=8, Hkv=1, D=256, cross=968),
                   dict(B=96, Sq=256, H=16, Hkv=16, D=72),
                   dict(B=16, Sq=1283, H=8, Hkv=4, D=256, causal_tail=515),
                   dict(B=4, Sq=4096, H=16, Hkv=8, D=128, causal_tail=4096)]:
            print(json.dumps(bench_attention(**kw, backward=True)), flush=True)
        for r in bench_membound():
            print(json.dumps(r), flush=True)


if __name__ == "__main__":
    main()
