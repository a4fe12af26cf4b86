"""Headline benchmark: pi0.5 training throughput (samples/s over the whole job) on N B200s.

Config = the full pi0.5 of the baseline definition: SigLIP-So400m/14 @224 x 3 cameras, Gemma-2B
backbone, Gemma-300M action expert, 200 prompt tokens, state 32, action chunk 50x32, knowledge
insulation, 256 FAST-style action tokens co-trained with the flow loss, bf16, batch 32 per GPU,
synthetic inputs, random-init weights.  One step = forward + backward + gradient sync + clip +
AdamW + parameter refresh.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|oracle] [--mode train|infer]

``--mode infer`` measures the second headline number instead: the p50 latency of one 10-step action chunk at batch 1.

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N``.
Rank 0 prints ONE JSON line.  ``--impl reference`` reports that the reference cannot be imported in
this image: its dependencies are not in the offline wheelhouse; ``--impl oracle`` runs this repository's plain-PyTorch/cuBLAS statement of
the same model (a library baseline, not the reference).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "oracle"])
    ap.add_argument("--batch", type=int, default=None,
                    help="per-GPU batch size (default: 32 for pi0.5, 16 for pi0.6: the baseline configs)")
    ap.add_argument("--comm", default="auto", choices=["auto", "p2p", "nccl"])
    ap.add_argument("--strategy", default="zero2")
    ap.add_argument("--tiny", action="store_true", help="small geometry (plumbing check, not a benchmark)")
    ap.add_argument("--mode", default="train", choices=["train", "infer"])
    ap.add_argument("--tp", type=int, default=1,
                    help="--model cosmos3: tensor-parallel width of the frozen backbone; must equal --gpus or 1")
    ap.add_argument("--cp", type=int, default=1,
                    help="--model pi07: context-parallel width (ranks that share every sequence); must equal --gpus "
                         "or 1")
    ap.add_argument("--model", default="pi05", choices=["pi05", "cosmos3", "pi06", "pi07"],
                    help="train mode: pi05 (headline) or pi06; infer mode: also cosmos3, the workload of the "
                         "reference's published B200 latency table")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end region (profiling runs only)")
    ap.add_argument("--train-vision", action="store_true",
                    help="train mode: also train the SigLIP tower (no frozen weights at all).  The default keeps the "
                         "policy config's own default, freeze_vision_encoder=true (reference "
                         "pi05/configuration_pi05.py:172): backbone, expert and every head train, the tower runs "
                         "forward only.  With the tower trained the step holds 166 GiB on one GPU at batch 32.")
    ap.add_argument("--dropout", type=float, default=0.1,
                    help="dropout after the attention output projection and the MLP (reference default 0.1, "
                         "pi05/configuration_pi05.py:148); printed in the config block")
    ap.add_argument("--ref-attn", default="sdpa", choices=["eager", "sdpa"],
                    help="--impl reference: the reference's attention_implementation (its docs recommend sdpa)")
    ap.add_argument("--ref-accum", type=int, default=1,
                    help="--impl reference: its gradient_accumulation_steps (doubled automatically when a pass of "
                         "the full per-GPU batch runs out of memory)")
    ap.add_argument("--ref-compile", default="on", choices=["on", "off"],
                    help="--impl reference: the reference's use_torch_compile (its pi0.5 default is on)")
    ap.add_argument("--kernel-table", default="", metavar="PATH",
                    help="train mode: after the warm-up, trace ONE step with the activity profiler, write the "
                         "per-kernel device-time shares to PATH and exit without a benchmark line")
    a = ap.parse_args()
    if a.batch is None:
        a.batch = {"pi06": 16, "pi07": 2, "cosmos3": 8}.get(a.model, 32)
    return a


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])), smax.append(float(f[2])), power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def build_policy_pi06(args, device):
    """pi0.6 training geometry: Gemma-3-4B backbone (34 layers, width 2560, 8 heads / 4 KV heads, head dim 256, MLP
    10240), SigLIP at 448x448 pooled to 256 tokens per camera, 3 cameras, the 1280-wide 34-layer action expert,
    256 prompt tokens, state 32, action chunk 50x32, knowledge insulation + 256 FAST tokens like pi0.5
    (reference ``policies/pi06/configuration_pi06.py:38-276``)."""
    import torch
    from opentau_b200.configs.types import FeatureType, PolicyFeature
    from opentau_b200.datasets.synthetic import SyntheticSpec, identity_stats
    from opentau_b200.policies.pi06.configuration_pi06 import PI06Config
    from opentau_b200.policies.pi06.modeling_pi06 import PI06Policy
    cams = 3
    res = (224, 224) if args.tiny else (448, 448)
    feats = {f"camera{i}": PolicyFeature(FeatureType.VISUAL, (3, *res)) for i in range(cams)}
    feats["state"] = PolicyFeature(FeatureType.STATE, (32,))
    kw = dict(chunk_size=50, n_action_steps=50, prompt_max_length=256, discrete_action_max_length=256,
              discrete_action_vocab_size=2048, dropout=args.dropout, knowledge_insulation=True, device=str(device),
              freeze_vision_encoder=not args.train_vision, train_expert_only=False, resize_imgs_with_padding=res,
              input_features=feats, output_features={"actions": PolicyFeature(FeatureType.ACTION, (32,))})
    vocab = 262208
    spec = SyntheticSpec(batch_size=args.batch, num_cams=cams, resolution=res, prompt_len=256, vocab_size=vocab,
                         state_dim=32, action_dim=32, chunk_size=50, discrete_action_len=256,
                         discrete_action_vocab=2048, image_dtype=torch.bfloat16)
    if args.tiny:
        kw.update(vlm=dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                           head_dim=64, intermediate_size=1024, vocab_size=1024, sliding_window_pattern=2),
                  expert=dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                              head_dim=64, intermediate_size=512, vocab_size=1024),
                  vision=dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4),
                  vlm_config={"tokens_per_image_side": 8}, discrete_action_vocab_size=256, proj_width=128)
        spec.vocab_size, spec.discrete_action_vocab = 1024, 256
    cfg = PI06Config(**kw)
    torch.manual_seed(1234)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)       # 5.6 B parameters: build them in bf16, not fp32 first
    try:
        with torch.device(device):
            policy = PI06Policy(cfg, per_dataset_stats=[identity_stats()])
    finally:
        torch.set_default_dtype(prev)
    policy.to(torch.bfloat16)
    policy.train()
    return policy, spec, cfg


def build_policy_pi07(args, device):
    """Long-context pi0.7 controller: SpaceTime-SigLIP video encoder over 16 frames x 3 cameras at 448x448, every
    frame's 256 pooled tokens kept in the decoder (12 288 vision tokens as 48 frame blocks), Gemma-3-4B backbone, a
    1024-wide ("300 M") action expert, 128 prompt tokens, a 128-token plan segment (the subtask text of the
    planner), action chunk 50x32, knowledge insulation + FAST tokens.  The decoder sequence is split over
    ``--cp`` ranks (``parallel/cp.py``)."""
    import torch
    from opentau_b200.configs.types import FeatureType, PolicyFeature
    from opentau_b200.datasets.synthetic import SyntheticSpec, identity_stats
    from opentau_b200.policies.factory import make_policy, make_policy_config
    cams, frames = 3, (3 if args.tiny else 16)
    res = (224, 224) if args.tiny else (448, 448)
    feats = {f"camera{i}": PolicyFeature(FeatureType.VISUAL, (3, *res)) for i in range(cams)}
    feats["state"] = PolicyFeature(FeatureType.STATE, (32,))
    fast = 8 if args.tiny else 32
    kw = dict(n_obs_steps=frames, chunk_size=50, n_action_steps=50, prompt_max_length=128, response_max_length=128,
              discrete_action_max_length=fast, discrete_action_vocab_size=2048, dropout=args.dropout,
              knowledge_insulation=True, device=str(device), freeze_vision_encoder=not args.train_vision,
              train_expert_only=False, resize_imgs_with_padding=res, keep_history_tokens=True,
              input_features=feats, output_features={"actions": PolicyFeature(FeatureType.ACTION, (32,))},
              expert=dict(hidden_size=1024, intermediate_size=4096), proj_width=1024)
    vocab = 262208
    if args.tiny:
        kw.update(vlm=dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                           head_dim=64, intermediate_size=1024, vocab_size=1024, sliding_window_pattern=2),
                  expert=dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                              head_dim=64, intermediate_size=512, vocab_size=1024),
                  vision=dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4),
                  vlm_config={"tokens_per_image_side": 8}, discrete_action_vocab_size=256, proj_width=128,
                  spacetime_layer_stride=2, prompt_max_length=16, response_max_length=8)
        vocab = 1024
    cfg = make_policy_config("pi07_low_level", **kw)
    spec = SyntheticSpec(batch_size=args.batch, num_cams=cams, resolution=res, prompt_len=cfg.prompt_max_length,
                         vocab_size=vocab, state_dim=32, action_dim=32, chunk_size=50, discrete_action_len=fast,
                         discrete_action_vocab=cfg.discrete_action_vocab_size, image_dtype=torch.bfloat16)
    spec.history, spec.response_len = frames, cfg.response_max_length
    torch.manual_seed(1234)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(device):
            policy = make_policy(cfg, per_dataset_stats=[identity_stats()])
    finally:
        torch.set_default_dtype(prev)
    policy.to(torch.bfloat16)
    policy.train()
    return policy, spec, cfg


def pi07_batch(spec, device, seed: int, pinned: bool):
    """Synthetic pi0.7 batch: the standard one plus a frame axis on cameras / state and the plan tokens."""
    import torch
    from opentau_b200.datasets.synthetic import make_synthetic_batch
    b = make_synthetic_batch(spec, device="cpu", seed=seed)
    g = torch.Generator().manual_seed(seed + 17)
    T = spec.history
    for k in [k for k in b if k.startswith("camera")]:
        img = b[k]
        b[k] = (img[:, None] * torch.linspace(0.5, 1.0, T).view(1, T, 1, 1, 1).to(img.dtype)).contiguous()
    b["state"] = b["state"][:, None].repeat(1, T, 1).contiguous()
    b["response_tokens"] = torch.randint(3, spec.vocab_size, (spec.batch_size, spec.response_len), generator=g)
    b["response_masks"] = torch.ones(spec.batch_size, spec.response_len, dtype=torch.bool)
    if pinned:
        b = {k: (v.pin_memory() if hasattr(v, "pin_memory") else v) for k, v in b.items()}
    return {k: (v.to(device) if hasattr(v, "to") else v) for k, v in b.items()}


def build_policy_cosmos3(args, device):
    """cosmos3 training geometry: frozen Qwen3-VL-32B-shaped backbone (64 layers, width 5120, 64 heads / 8 KV heads,
    head dim 128, SwiGLU 25600), 2 cameras at 448x448 (patch 16, 2x2 merge: 196 tokens each), 128 prompt tokens,
    a trainable 24-layer 1024-wide action expert that reads the last backbone layer (``condition_on_layer=63``),
    state 32, action chunk 50x32.  ``--tp N`` shards the backbone over the N ranks with the GEMM -> reduce-scatter
    and all-gather -> GEMM kernels (``parallel/tp.py``); the expert stays data parallel."""
    from opentau_b200.scripts.benchmark_inference import build_cosmos3
    policy, spec, cfg = build_cosmos3(2, 128, device, tiny=args.tiny, num_steps=10, image=448, expert_layers=24,
                                      condition_on_layer=63, batch=args.batch, train=True, dropout=args.dropout)
    spec.discrete_action_len = 0
    return policy, spec, cfg


def enable_tp(args, policy, device, world):
    if args.tp <= 1:
        return
    if args.tp != world:
        raise SystemExit("--tp must equal the number of ranks (one tensor-parallel group per node) or 1")
    from opentau_b200.parallel.tp import TensorParallel
    policy.enable_tensor_parallel(TensorParallel(device), free_replicated_weights=True)


def build_policy(args, device):
    if args.model == "cosmos3":
        return build_policy_cosmos3(args, device)
    if args.model == "pi06":
        return build_policy_pi06(args, device)
    if args.model == "pi07":
        return build_policy_pi07(args, device)
    import torch
    from opentau_b200.configs.types import FeatureType, PolicyFeature
    from opentau_b200.datasets.synthetic import SyntheticSpec, identity_stats
    from opentau_b200.policies.pi05.configuration_pi05 import PI05Config
    from opentau_b200.policies.pi05.modeling_pi05 import PI05Policy

    cams = 3
    feats = {f"camera{i}": PolicyFeature(FeatureType.VISUAL, (3, 224, 224)) for i in range(cams)}
    feats["state"] = PolicyFeature(FeatureType.STATE, (32,))
    kw = dict(chunk_size=50, n_action_steps=50, prompt_max_length=200, discrete_action_max_length=256,
              discrete_action_vocab_size=2048, dropout=args.dropout, knowledge_insulation=True, device=str(device),
              freeze_vision_encoder=not args.train_vision, train_expert_only=False,
              input_features=feats, output_features={"actions": PolicyFeature(FeatureType.ACTION, (32,))})
    spec = SyntheticSpec(batch_size=args.batch, num_cams=cams, prompt_len=200, vocab_size=257152, state_dim=32,
                         action_dim=32, chunk_size=50, discrete_action_len=256, discrete_action_vocab=2048,
                         image_dtype=torch.bfloat16)
    if args.tiny:
        kw.update(vlm=dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1,
                           head_dim=64, intermediate_size=1024, vocab_size=1024),
                  expert=dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1,
                              head_dim=64, intermediate_size=512, vocab_size=1024),
                  vision=dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4),
                  discrete_action_vocab_size=256)
        spec.vocab_size, spec.discrete_action_vocab = 1024, 256
    cfg = PI05Config(**kw)
    torch.manual_seed(1234)
    with torch.device(device):
        policy = PI05Policy(cfg, per_dataset_stats=[identity_stats()])
    policy.to(torch.bfloat16)
    policy.train()
    return policy, spec, cfg


def run_infer(args, device, rank, world, local_rank, use_cuda) -> int:
    """Second headline metric: p50 latency of one 10-step flow-matching action chunk (pi0.5 full, batch 1, three
    cameras, 200 prompt tokens) through ``policy.sample_actions``.  Every rank serves its own replica; the reported
    value is the slowest rank's median.  The device-timed region is the call alone on resident inputs; the end-to-end
    region adds the pinned-host -> device copy of the observation and the device -> host read of the actions."""
    import torch
    import torch.distributed as dist
    from opentau_b200.ops import cuda_ops
    from opentau_b200.scripts.benchmark_inference import BUILDERS, summarize

    # published by the reference for this exact cosmos3 workload on 1 x B200 with torch.compile reduce-overhead
    # (docs/source/tutorials/benchmarking.rst:437-510): p50 106.86 ms
    published_p50 = {"cosmos3": 106.86}.get(args.model)
    prompt_len = 64 if args.model == "cosmos3" else 200
    num_steps = 5 if args.model == "pi06" else 10          # each policy's reference default
    if args.model == "cosmos3" and args.tp > 1:
        # the 8-GPU serving geometry: 2 cameras at 448x448, 128 prompt tokens, 24-layer expert on backbone layer 63,
        # backbone tensor parallel over the ranks, one observation per rank
        policy, batch = BUILDERS["cosmos3"](2, 128, device, tiny=args.tiny, num_steps=num_steps, image=448,
                                            expert_layers=24, condition_on_layer=63)
        enable_tp(args, policy, device, world)
    else:
        policy, batch = BUILDERS[args.model](3, prompt_len, device, tiny=args.tiny, num_steps=num_steps)
    # with a tensor-parallel backbone the prefix pass runs eagerly (its kernels carry a per-call epoch and it contains
    # collectives) and the expert's Euler loop behind it is replayed from a graph
    use_graphs = use_cuda and args.impl == "ours"
    if use_graphs:
        policy.enable_cuda_graphs(True)
    host = {k: (v.cpu().pin_memory() if use_cuda else v.cpu()) for k, v in batch.items() if hasattr(v, "cpu")}
    h2d_bytes = sum(v.numel() * v.element_size() for v in host.values())

    def sync():
        if world > 1:
            dist.barrier()
        if use_cuda:
            torch.cuda.synchronize()

    def one(e2e: bool) -> float:
        if use_cuda:
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        b = {k: v.to(device, non_blocking=True) for k, v in host.items()} if e2e else batch
        out = policy.sample_actions(b)
        if e2e:
            out = out.float().cpu()                      # device -> host read of the action chunk
        if use_cuda:
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1), out
        return (time.perf_counter() - t0) * 1e3, out

    for _ in range(max(args.warmup, 3)):
        one(False)
    if use_cuda and args.impl == "ours":
        cuda_ops.check_status()
    sampler = ClockSampler(local_rank)
    if rank == 0 and use_cuda:
        sampler.start()
    launches0 = cuda_ops.launch_count
    sync()
    dev_ms = [one(False)[0] for _ in range(args.steps)]
    sync()
    launches = cuda_ops.launch_count - launches0
    one(True)
    sync()
    res = [one(True) for _ in range(args.steps)]
    sync()
    e2e_ms, out = [r[0] for r in res], res[-1][1]
    clocks = sampler.stop() if (rank == 0 and use_cuda) else {}
    d2h_bytes = out.numel() * out.element_size()
    stats = torch.tensor([summarize(dev_ms)["p50_ms"], summarize(e2e_ms)["p50_ms"], sum(dev_ms) / len(dev_ms)],
                         dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    if rank == 0:
        n_params = sum(p.numel() for p in policy.parameters())
        print(json.dumps({
            "metric": f"{args.model} p50 {num_steps}-step action-chunk latency", "value": round(float(stats[0]), 3),
            "unit": "ms",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(float(stats[2]), 3), "higher_is_better": False, "scaling": "weak",
            "vs_baseline": (round(float(stats[0]) / published_p50, 4) if published_p50 and not args.tiny else None),
            "dtype": "bf16", "data": "synthetic", "impl": args.impl,
            "config": {"model": ("tiny (plumbing)" if args.tiny else
                                 "pi0.5 full (SigLIP-So400m/14@224 x3 cams, Gemma-2B, Gemma-300M expert)"
                                 if args.model == "pi05" else
                                 "pi0.6 (Gemma-3-4B backbone, SigLIP @448 x3 cams pooled to 256 tokens each, "
                                 "1280-wide 34-layer expert)" if args.model == "pi06" else
                                 "cosmos3 (Qwen3-VL-32B-shaped backbone sharded over the ranks, 24-layer expert on "
                                 "backbone layer 63, 2 cams @448, 128 prompt tokens)" if args.tp > 1 else
                                 "cosmos3 (Qwen3-VL-32B-shaped backbone, 64-layer 0.9B expert, 3 cams @224, "
                                 "prompt <= 64 tokens)"),
                       "global_batch": world,
                       "parallelism": f"tp{args.tp}, one observation per rank" if args.tp > 1 else f"replica x{world}",
                       "params": n_params, "denoise_steps": num_steps, "action_chunk": "50x32",
                       "cuda_graph": bool(use_graphs), "tensor_parallel": args.tp,
                       "l2": "each call streams every bf16 weight once (GBs, far more than the 126 MB L2); no "
                             "explicit flush"},
            "clocks": clocks,
            "e2e": {"value": round(float(stats[1]), 3), "unit": "ms", "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": d2h_bytes},
            "gpu_launches": launches,
        }))
    return 0


def write_kernel_table(path: str, step, sync, top: int = 60) -> None:
    """Trace one call of ``step`` with the CUDA activity profiler and write device time per kernel name.

    The figures are shares of one traced step (tracing perturbs the absolute time); the benchmark number is
    never taken from such a run.
    """
    import collections

    import torch
    from torch.profiler import ProfilerActivity, profile

    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        e0.record()
        step()
        e1.record()
        sync()
    agg = collections.defaultdict(lambda: [0, 0.0])
    for ev in prof.events():
        if ev.device_type == torch.autograd.DeviceType.CUDA:
            a = agg[ev.name[:120]]
            a[0] += 1
            a[1] += ev.device_time_total
    total = sum(v[1] for v in agg.values())
    ours = sum(v[1] for k, v in agg.items() if "otb" in k)
    n_all = sum(v[0] for v in agg.values())
    lines = [f"traced step {e0.elapsed_time(e1):.1f} ms between events; {n_all} device activities, "
             f"{total / 1e3:.1f} ms summed device time; kernels of this repository (otb::*) "
             f"{ours / 1e3:.1f} ms = {100 * ours / max(total, 1e-9):.1f} %"]
    for name, (n, t) in sorted(agg.items(), key=lambda kv: -kv[1][1])[:top]:
        lines.append(f"{t / 1e3:9.2f} ms {100 * t / total:5.1f} % n={n:5d} {t / n:9.1f} us  {name}")
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")
    print(lines[0])


def main():
    args = parse_args()
    if args.impl == "reference":
        # the reference's launcher default (scripts/launch.py:27-34); must be set before CUDA is initialised
        os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
        # torch.compile (the reference's default for pi0.5) builds host code with OpenMP; the image's CXX points
        # at a compiler wrapper without libgomp.spec, the system compiler has it
        if os.path.exists("/usr/bin/g++") and os.path.exists("/usr/bin/gcc"):
            os.environ["CXX"], os.environ["CC"] = "/usr/bin/g++", "/usr/bin/gcc"
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
        import reference_arm
        args.clock_sampler = ClockSampler
        if args.mode == "infer":
            return reference_arm.run_infer(args)
        return reference_arm.run_train(args)
    if args.impl == "oracle":
        os.environ["OPENTAU_B200_ORACLE"] = "1"

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("for --gpus N > 1 launch through torch.distributed.run with N ranks")
    use_cuda = torch.cuda.is_available()
    device = torch.device(f"cuda:{local_rank}" if use_cuda else "cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl" if use_cuda else "gloo", device_id=device if use_cuda else None)

    if args.mode == "infer":
        rc = run_infer(args, device, rank, world, local_rank, use_cuda)
        if world > 1:
            dist.destroy_process_group()
        return rc

    from opentau_b200.datasets.synthetic import make_synthetic_batch
    from opentau_b200.parallel.engine import OptimHyper
    from opentau_b200.parallel.fsdp import make_engine

    policy, spec, cfg = build_policy(args, device)
    if args.model == "pi07" and args.cp > 1:
        if args.cp != world:
            raise SystemExit("--cp must equal the number of ranks (one context-parallel group per node) or 1")
        from opentau_b200.parallel.cp import ContextParallel
        policy.model.context_parallel = ContextParallel(device)
    if args.model == "cosmos3":
        enable_tp(args, policy, device, world)
    engine = make_engine(policy, OptimHyper(lr=cfg.optimizer_lr, betas=tuple(cfg.optimizer_betas),
                                            eps=cfg.optimizer_eps, weight_decay=cfg.optimizer_weight_decay,
                                            grad_clip_norm=10.0),
                         device=device, strategy=args.strategy,
                         comm=("nccl" if args.impl == "oracle" else args.comm))
    n_params = sum(p.numel() for p in policy.parameters())

    # host batches in pinned memory (distinct per step so no step reuses a cached input)
    n_host = 4
    if args.model == "pi07":
        host = [pi07_batch(spec, "cpu", 1000 * rank + i, use_cuda) for i in range(n_host)]
    else:
        host = [make_synthetic_batch(spec, device="cpu", seed=1000 * rank + i, pinned=use_cuda)
                for i in range(n_host)]
    dev_batches = [{k: v.to(device) for k, v in b.items()} for b in host[:2]]
    h2d_bytes = sum(v.numel() * v.element_size() for v in host[0].values())

    def sync():
        if world > 1:
            dist.barrier()
        if use_cuda:
            torch.cuda.synchronize()

    from opentau_b200.ops import cuda_ops

    def run_device_only(n):
        for i in range(n):
            engine.train_step(dev_batches[i % 2])

    def run_e2e(n):
        last = None
        for i in range(n):
            hb = host[i % n_host]
            b = {k: v.to(device, non_blocking=True) for k, v in hb.items()}
            out = engine.train_step(b)
            last = float(out["loss"].item())  # device -> host read of the step's result
        return last

    def timed(fn, n):
        sync()
        if use_cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            res = fn(n)
            e1.record()
            sync()
            ms = e0.elapsed_time(e1)
        else:
            t0 = time.perf_counter()
            res = fn(n)
            ms = (time.perf_counter() - t0) * 1e3
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), res

    first = engine.train_step(dev_batches[0])
    first_grad_norm = float(first["grad_norm"])      # same seeds and batches for every --comm: comparable across runs
    run_device_only(args.warmup - 1)
    if use_cuda and args.impl == "ours":
        cuda_ops.check_status()
        engine.check()
    if args.kernel_table:
        if rank == 0:
            # local synchronisation only: the other ranks run the same step without the tracer around it
            write_kernel_table(args.kernel_table, lambda: run_device_only(1), torch.cuda.synchronize)
        else:
            run_device_only(1)
        if world > 1:
            dist.destroy_process_group()
        return 0
    sampler = ClockSampler(local_rank)
    if rank == 0 and use_cuda:
        sampler.start()
    launches0 = cuda_ops.launch_count
    ms_dev, _ = timed(run_device_only, args.steps)
    launches = cuda_ops.launch_count - launches0
    if args.no_e2e:
        ms_e2e, last_loss = float("nan"), None
    else:
        run_e2e(1)
        ms_e2e, last_loss = timed(run_e2e, args.steps)
    clocks = sampler.stop() if (rank == 0 and use_cuda) else {}
    if use_cuda and args.impl == "ours":
        cuda_ops.check_status()
        engine.check()
    # cross-rank evidence that the replicas stayed identical through the timed region
    checksum = engine.param_checksum()
    sums = [checksum.clone() for _ in range(world)]
    if world > 1:
        dist.all_gather(sums, checksum)
    sums = [float(x.item()) for x in sums]
    replicas_equal = all(x == sums[0] for x in sums)

    global_batch = args.batch * world
    value = global_batch * args.steps / (ms_dev / 1e3)
    e2e_value = global_batch * args.steps / (ms_e2e / 1e3)
    if rank == 0:
        peak_gb = torch.cuda.max_memory_allocated() / 2**30 if use_cuda else 0.0
        # the symmetric (peer-mapped) buffers are allocated outside the caching allocator: the device-wide figure
        # is the one that compares strategies
        free_b, total_b = torch.cuda.mem_get_info() if use_cuda else (0, 0)
        print(json.dumps({
            "metric": f"{ {'pi06': 'pi0.6', 'pi07': 'pi0.7 long-context', 'cosmos3': 'cosmos3'}.get(args.model, 'pi0.5') } train samples/s/box", "value": round(value, 3),
            "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_dev / args.steps, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": args.impl,
            "config": {"model": ("tiny (plumbing)" if args.tiny else
                                 "pi0.6 (SigLIP-So400m/14@448 x3 cams pooled to 256 tokens each, Gemma-3-4B, 1280-wide "
                                 "34-layer expert)" if args.model == "pi06" else
                                 "pi0.7 controller, long context (SpaceTime SigLIP, 16 frames x 3 cams x 256 tokens "
                                 "kept in the decoder, Gemma-3-4B, 1024-wide expert, 128 prompt + 128 plan tokens)"
                                 if args.model == "pi07" else
                                 "cosmos3 (frozen Qwen3-VL-32B-shaped backbone, 2 cams @448 -> 196 tokens each, 128 "
                                 "prompt tokens, trainable 24-layer 1024-wide expert on backbone layer 63)"
                                 if args.model == "cosmos3" else
                                 "pi0.5 full (SigLIP-So400m/14@224 x3 cams, Gemma-2B, Gemma-300M expert)"),
                       "global_batch": global_batch,
                       "seq_len": (getattr(spec, "history", 1) * 3 * 256 + spec.prompt_len + getattr(spec, "response_len", 0)
                                   + spec.discrete_action_len + 3) if args.model == "pi07"
                       else 3 * 256 + spec.prompt_len + 3 + 256,
                       "parallelism": f"dp{world}-{engine.strategy}-{engine.comm}" + (
                           f"+cp{args.cp}" if args.model == "pi07" else f"+tp{args.tp}" if args.model == "cosmos3"
                           else ""), "params": n_params,
                       "knowledge_insulation": True, "fast_tokens": spec.discrete_action_len, "action_chunk": "50x32",
                       "dropout": args.dropout,
                       "frozen_weights": "none" if args.train_vision else "SigLIP tower (policy default "
                                                                           "freeze_vision_encoder=true)",
                       "trainable_params": sum(p.numel() for p in policy.parameters() if p.requires_grad),
                       "l2": "per-step working set (tens of GB of activations) far exceeds the 126 MB L2; "
                             "no explicit flush", "peak_mem_gib": round(peak_gb, 2),
                       "device_mem_in_use_gib": round((total_b - free_b) / 2**30, 2)},
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 3), "unit": "samples/s", "ms_per_step": round(ms_e2e / args.steps, 3),
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4, "last_loss": last_loss},
            "gpu_launches": launches,
            "checks": {"replicas_equal": replicas_equal, "param_checksum": sums[0],
                       "first_step_grad_norm": round(first_grad_norm, 4),
                       "overlap_grad_reduce": bool(getattr(engine, "overlap", False))},
        }))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
