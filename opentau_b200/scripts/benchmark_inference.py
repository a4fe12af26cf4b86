"""Action-chunk latency benchmark: ``sample_actions`` on a fixed observation, batch 1 by default.

Counterpart of the reference script (OpenTau ``src/opentau/scripts/benchmark_inference.py:153-331``): warm-up
calls, then timed calls each bracketed by a device synchronise, reporting mean / std / p50 / p95 / p99.  The
"compiled" arm of the reference (``torch.compile`` + CUDA graphs) corresponds here to ``--graphs`` (replay of
the captured sampler); ``--no-graphs`` is the eager arm.  Environment knobs kept: ``BENCH_N_WARMUP``,
``BENCH_N_TIMED``, ``BENCH_N_CANDIDATES``, ``BENCH_OUTPUT_DIR``, ``BENCH_NO_COMPILE`` (eager only) and
``BENCH_COMPILE_MODE`` (any value: graph replay).

    python -m opentau_b200.scripts.benchmark_inference [--policy pi05] [--cams 3] [--prompt-len 200] [--graphs]
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import time
from pathlib import Path

import torch

BENCHMARK_PROMPT = "pick up the red block and place it in the bin"


def summarize(ms: list[float]) -> dict:
    s = sorted(ms)

    def pct(p: float) -> float:
        k = (len(s) - 1) * p
        lo, hi = int(k), min(int(k) + 1, len(s) - 1)
        return s[lo] + (s[hi] - s[lo]) * (k - lo)

    return {"n": len(s), "mean_ms": statistics.fmean(s), "std_ms": statistics.pstdev(s) if len(s) > 1 else 0.0,
            "p50_ms": pct(0.5), "p95_ms": pct(0.95), "p99_ms": pct(0.99), "min_ms": s[0], "max_ms": s[-1]}


def build_pi05(cams: int, prompt_len: int, device, tiny: bool = False, num_steps: int = 10,
               depth: int | None = None):
    from ..configs.types import FeatureType, PolicyFeature
    from ..datasets.synthetic import SyntheticSpec, identity_stats, make_synthetic_batch
    from ..policies.pi05.configuration_pi05 import PI05Config
    from ..policies.pi05.modeling_pi05 import PI05Policy
    feats = {f"camera{i}": PolicyFeature(FeatureType.VISUAL, (3, 224, 224)) for i in range(cams)}
    feats["state"] = PolicyFeature(FeatureType.STATE, (32,))
    kw = dict(chunk_size=50, n_action_steps=50, prompt_max_length=prompt_len, num_steps=num_steps, dropout=0.0,
              device=str(device), input_features=feats,
              output_features={"actions": PolicyFeature(FeatureType.ACTION, (32,))})
    spec = SyntheticSpec(batch_size=1, num_cams=cams, prompt_len=prompt_len, vocab_size=257152, state_dim=32,
                         action_dim=32, chunk_size=50, image_dtype=torch.bfloat16)
    if tiny:
        kw.update(vlm=dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1,
                           head_dim=64, intermediate_size=1024, vocab_size=1024),
                  expert=dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1,
                              head_dim=64, intermediate_size=512, vocab_size=1024),
                  vision=dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4))
        spec.vocab_size = 1024
    cfg = PI05Config(**kw)
    torch.manual_seed(0)
    with torch.device(device):
        policy = PI05Policy(cfg, per_dataset_stats=[identity_stats()])
    policy.to(device).to(torch.bfloat16).eval()
    batch = make_synthetic_batch(spec, device=device, seed=3)
    return policy, batch


def build_cosmos3(cams: int, prompt_len: int, device, tiny: bool = False, num_steps: int = 10,
                  depth: int | None = None, image: int = 224, expert_layers: int | None = None,
                  condition_on_layer: int | None = None, batch: int = 1, train: bool = False, dropout: float = 0.0):
    """The workload of the reference's published cosmos3 latency table (``docs/source/tutorials/benchmarking.rst:
    437-510``): the full 64-layer Qwen3-VL-32B-shaped backbone, the 64-layer action expert reading a per-layer KV
    cache, ``cams`` cameras at 224x224, a prompt capped at ``prompt_len`` tokens, a 50-action chunk.  Weights are
    random (no checkpoint offline)."""
    from ..configs.types import FeatureType, PolicyFeature
    from ..datasets.synthetic import SyntheticSpec, identity_stats, make_synthetic_batch
    from ..policies.cosmos3.configuration_cosmos3 import Cosmos3Config
    from ..policies.cosmos3.modeling_cosmos3 import Cosmos3Policy
    if tiny:
        image = 224
    feats = {f"camera{i}": PolicyFeature(FeatureType.VISUAL, (3, image, image)) for i in range(cams)}
    feats["state"] = PolicyFeature(FeatureType.STATE, (32,))
    kw = dict(chunk_size=50, n_action_steps=50, prompt_max_length=prompt_len, num_steps=num_steps, dropout=dropout,
              device=str(device), input_features=feats, load_pretrained_backbone=False, image_resize=image,
              output_features={"actions": PolicyFeature(FeatureType.ACTION, (32,))})
    if expert_layers is not None:
        # an expert whose depth differs from the backbone's reads ONE backbone layer's keys / values
        # (reference cosmos3/qwen3vl_with_expert.py:405-432)
        kw.update(expert_num_hidden_layers=expert_layers,
                  condition_on_layer=condition_on_layer if condition_on_layer is not None else -1)
    vocab = 151936
    if tiny:
        kw.update(backbone=dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                                head_dim=32, intermediate_size=256, vocab_size=512, mrope_sections=(6, 5, 5)),
                  vision=dict(hidden_size=64, depth=2, num_heads=4, intermediate_size=128, out_hidden_size=128,
                              num_position_embeddings=256, deepstack_visual_indexes=(0,)),
                  expert_hidden_size=64, expert_intermediate_size=128, expert_num_hidden_layers=2,
                  expert_num_attention_heads=4, expert_num_key_value_heads=2, expert_head_dim=32, proj_width=64,
                  expert_adarms_cond_dim=32)
        vocab = 512
    if depth is not None:                       # same layers, fewer of them: a small case for profiling
        kw.update(backbone=dict(num_hidden_layers=depth), expert_num_hidden_layers=depth)
    if tiny and expert_layers is not None:
        kw.update(expert_num_hidden_layers=3, condition_on_layer=1)
    cfg = Cosmos3Config(**kw)
    spec = SyntheticSpec(batch_size=batch, num_cams=cams, resolution=(image, image), prompt_len=prompt_len,
                         vocab_size=vocab, state_dim=32, action_dim=32, chunk_size=50, image_dtype=torch.bfloat16)
    torch.manual_seed(0)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)     # 33 B parameters: never materialise them in fp32
    try:
        with torch.device(device):
            policy = Cosmos3Policy(cfg, per_dataset_stats=[identity_stats()])
    finally:
        torch.set_default_dtype(prev)
    policy.to(device).to(torch.bfloat16)
    policy.train() if train else policy.eval()
    if train:
        return policy, spec, cfg
    return policy, make_synthetic_batch(spec, device=device, seed=3)


def build_pi06(cams: int, prompt_len: int, device, tiny: bool = False, num_steps: int = 5,
               depth: int | None = None):
    """pi0.6 at its reference geometry (``src/opentau/policies/pi06/configuration_pi06.py:38-276``): Gemma-3-4B
    backbone, ``cams`` cameras at 448x448 pooled to 256 tokens each, the 1280-wide 34-layer action expert, a
    50-action chunk in 5 flow-matching steps (the reference quotes the model card's "~63 ms per chunk on an H100"
    for this shape).  Random weights."""
    from ..configs.types import FeatureType, PolicyFeature
    from ..datasets.synthetic import SyntheticSpec, identity_stats, make_synthetic_batch
    from ..policies.pi06.configuration_pi06 import PI06Config
    from ..policies.pi06.modeling_pi06 import PI06Policy
    res = (224, 224) if tiny else (448, 448)
    feats = {f"camera{i}": PolicyFeature(FeatureType.VISUAL, (3, *res)) for i in range(cams)}
    feats["state"] = PolicyFeature(FeatureType.STATE, (32,))
    kw = dict(chunk_size=50, n_action_steps=50, prompt_max_length=prompt_len, num_steps=num_steps, dropout=0.0,
              device=str(device), input_features=feats, resize_imgs_with_padding=res,
              output_features={"actions": PolicyFeature(FeatureType.ACTION, (32,))})
    vocab = 262208
    if tiny:
        kw.update(vlm=dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                           head_dim=64, intermediate_size=1024, vocab_size=1024, sliding_window_pattern=2),
                  expert=dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                              head_dim=64, intermediate_size=512, vocab_size=1024),
                  vision=dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4),
                  vlm_config={"tokens_per_image_side": 8})
        vocab = 1024
    cfg = PI06Config(**kw)
    spec = SyntheticSpec(batch_size=1, num_cams=cams, resolution=res, prompt_len=prompt_len, vocab_size=vocab,
                         state_dim=32, action_dim=32, chunk_size=50, image_dtype=torch.bfloat16)
    torch.manual_seed(0)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(device):
            policy = PI06Policy(cfg, per_dataset_stats=[identity_stats()])
    finally:
        torch.set_default_dtype(prev)
    policy.to(device).to(torch.bfloat16).eval()
    batch = make_synthetic_batch(spec, device=device, seed=3)
    return policy, batch


BUILDERS = {"pi05": build_pi05, "cosmos3": build_cosmos3, "pi06": build_pi06}


def run(policy, batch, n_warmup: int, n_timed: int, n_candidates: int = 1) -> dict:
    dev = batch["state"].device
    cuda = dev.type == "cuda"
    times = []
    for i in range(n_warmup + n_timed):
        if cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = policy.sample_actions(batch, n_candidates=n_candidates)
        if cuda:
            torch.cuda.synchronize()
        if i >= n_warmup:
            times.append((time.perf_counter() - t0) * 1e3)
    assert torch.isfinite(out).all()
    return summarize(times)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--policy", default="pi05", choices=sorted(BUILDERS))
    ap.add_argument("--cams", type=int, default=3)
    ap.add_argument("--prompt-len", type=int, default=None, help="default: 200 (pi05), 64 (cosmos3)")
    ap.add_argument("--num-steps", type=int, default=10)
    ap.add_argument("--graphs", dest="graphs", action="store_true", default=True)
    ap.add_argument("--no-graphs", dest="graphs", action="store_false")
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--depth", type=int, default=None, help="cosmos3: truncate backbone and expert to this many layers")
    args = ap.parse_args(argv)
    # the reference's knobs: BENCH_NO_COMPILE=1 is its eager arm; any BENCH_COMPILE_MODE maps to graph replay here
    if os.environ.get("BENCH_NO_COMPILE", "0").lower() in ("1", "true"):
        args.graphs = False
    elif os.environ.get("BENCH_COMPILE_MODE"):
        args.graphs = True
    n_warmup = int(os.environ.get("BENCH_N_WARMUP", "5"))
    n_timed = int(os.environ.get("BENCH_N_TIMED", "50"))
    n_cand = int(os.environ.get("BENCH_N_CANDIDATES", "1"))
    device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    if args.prompt_len is None:
        args.prompt_len = 64 if args.policy == "cosmos3" else 200
    policy, batch = BUILDERS[args.policy](args.cams, args.prompt_len, device, args.tiny, args.num_steps, args.depth)
    if n_cand > 1:
        # the parameter-free consensus selector; it cannot rank two candidates, so BENCH_N_CANDIDATES=2 fails here
        from ..policies.candidates import MEDOID, configure_candidates
        configure_candidates(policy, n_cand, MEDOID, device=device)
    rec = {"policy": args.policy, "device": torch.cuda.get_device_name(0) if device.type == "cuda" else "cpu",
           "dtype": "bf16", "num_steps": args.num_steps, "n_candidates": n_cand, "cams": args.cams,
           "prompt_len": args.prompt_len}
    if device.type == "cuda":
        from ..ops import cuda_ops
        policy.enable_cuda_graphs(False)
        rec["eager"] = run(policy, batch, n_warmup, n_timed, n_cand)
        if args.graphs:
            policy.enable_cuda_graphs(True)
            rec["cuda_graph"] = run(policy, batch, n_warmup, n_timed, n_cand)
        cuda_ops.check_status()
    else:
        rec["eager"] = run(policy, batch, 1, 3, n_cand)
    print(json.dumps(rec))
    out_dir = os.environ.get("BENCH_OUTPUT_DIR")
    if out_dir:
        Path(out_dir).mkdir(parents=True, exist_ok=True)
        (Path(out_dir) / f"benchmark_inference_{args.policy}.json").write_text(json.dumps(rec, indent=2))
    return rec


if __name__ == "__main__":
    main()
