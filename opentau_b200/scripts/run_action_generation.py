"""Action generation from one image and one instruction, timed over several flow-matching step counts
(reference ``src/opentau/scripts/run_action_generation.py:17-364``).

Action generation = one conditioning IMAGE + one language PROMPT -> an action chunk ``[chunk_size, action_dim]``; no
video in or out.  The reference script drives NVIDIA's 64 B Cosmos3-Super through a diffusers pipeline that exists only
on that library's main branch (and a hub download of ~129 GB); this one drives the framework's own cosmos3 policy
(``policies/cosmos3``: Qwen3-VL backbone + flow-matching expert) through the same interface and reports the same things:
one latency per step count (model loaded once, ``--warmup`` untimed calls first), the action tensor of the last run as
JSON, and a summary table.  The observation goes from pinned host memory to the device inside the timed region; on a GPU
the sampler is replayed from a CUDA graph per step count.

    python -m opentau_b200.scripts.run_action_generation --image frame.png --prompt "pick up the cup" \\
        --domain agibotworld --chunk-size 50 --steps 30,10,5 --warmup 1 --output action.json \\
        [--checkpoint <dir | repo@rev>] [--config_path policy_or_train_config.json]

Without ``--checkpoint`` the weights are randomly initialised (a timing run); ``--tiny`` shrinks the geometry for a
smoke run on a CPU.
"""

from __future__ import annotations

import argparse
import json
import time
from pathlib import Path

import numpy as np
import torch

#: embodiment -> action width (the reference's table: agibotworld 29, droid / franka 10, autonomous vehicle 9)
DOMAIN_ACTION_DIM = {"agibotworld": 29, "droid": 10, "franka": 10, "av": 9}


def parse_args(argv=None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--image", required=True, help="the conditioning observation (png / jpg)")
    p.add_argument("--prompt", default="Pickup items in the supermarket")
    p.add_argument("--domain", default="agibotworld", help=f"sets the action width: {DOMAIN_ACTION_DIM}")
    p.add_argument("--action-dim", type=int, default=None, help="overrides the domain's action width")
    p.add_argument("--chunk-size", type=int, default=50)
    p.add_argument("--num-inference-steps", type=int, default=30, help="flow-matching steps when --steps is empty")
    p.add_argument("--steps", default="", help="comma-separated step counts to sweep in one process, e.g. 30,10,5")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--warmup", type=int, default=0, help="untimed calls per step count before the timed one")
    p.add_argument("--repeats", type=int, default=1, help="timed calls per step count (the median is reported)")
    p.add_argument("--checkpoint", default=None, help="a cosmos3 checkpoint (directory or repo@rev in the local cache)")
    p.add_argument("--config_path", default=None, help="a policy or pipeline config to take the geometry from")
    p.add_argument("--device", default=None)
    p.add_argument("--no-graphs", action="store_true", help="issue every launch from Python")
    p.add_argument("--tiny", action="store_true", help="a few-layer geometry (smoke runs)")
    p.add_argument("--output", default="action.json")
    return p.parse_args(argv)


def load_image(path: str | Path, size: int) -> torch.Tensor:
    """``(1, 3, size, size)`` float in [0, 1], resized with aspect-preserving padding like the data pipeline."""
    from PIL import Image

    from .. import ops
    arr = np.asarray(Image.open(path).convert("RGB"), np.float32) / 255.0
    t = torch.from_numpy(arr).permute(2, 0, 1)[None]
    return ops.resize_with_pad(t, size, size, pad_value=0.0) if tuple(t.shape[-2:]) != (size, size) else t


def build_policy(args: argparse.Namespace, action_dim: int):
    from ..configs.types import FeatureType, PolicyFeature
    from ..datasets.synthetic import identity_stats
    from ..policies.factory import make_policy, make_policy_config
    if args.config_path:
        from ..configs import parser
        from ..configs.train import TrainPipelineConfig
        cfg = parser.parse_config(TrainPipelineConfig, [f"--config_path={args.config_path}"]).policy
    else:
        kw = dict(chunk_size=args.chunk_size, n_action_steps=args.chunk_size, device="cpu")
        if args.tiny:
            kw.update(image_resize=128, prompt_max_length=16, proj_width=64, expert_hidden_size=64,
                      expert_intermediate_size=128, expert_num_hidden_layers=2, expert_num_attention_heads=4,
                      expert_num_key_value_heads=2, expert_head_dim=32, expert_adarms_cond_dim=32,
                      backbone=dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                                    head_dim=32, intermediate_size=256, vocab_size=1024, mrope_sections=(6, 5, 5)),
                      vision=dict(hidden_size=64, depth=2, num_heads=4, intermediate_size=128,
                                  num_position_embeddings=64, deepstack_visual_indexes=(0, 1)))
        cfg = make_policy_config("cosmos3", **kw)
    if cfg.type not in ("cosmos3", "cosmos3_nano"):
        raise ValueError(f"action generation drives the cosmos3 family, the configuration names {cfg.type!r}")
    if not cfg.input_features:
        size = int(getattr(cfg, "image_resize", 224) or 224)
        cfg.input_features = {"camera0": PolicyFeature(FeatureType.VISUAL, (3, size, size)),
                              "state": PolicyFeature(FeatureType.STATE, (cfg.max_state_dim,))}
        cfg.output_features = {"actions": PolicyFeature(FeatureType.ACTION, (action_dim,))}
    if args.checkpoint:
        cfg.pretrained_path = args.checkpoint
        return make_policy(cfg), cfg
    # statistics sized to the BOUND features (the action feature has the domain's width, not the padded one)
    stats = identity_stats(cfg.input_features["state"].shape[0], cfg.output_features["actions"].shape[0])
    return make_policy(cfg, per_dataset_stats=[stats]), cfg


def generate(policy, batch_host: dict, device: torch.device, n_steps: int, seed: int) -> tuple[torch.Tensor, float]:
    """One timed call: pinned observation -> device, ``n_steps`` Euler steps, action chunk back on the host."""
    cfg = policy.config
    cfg.num_steps = n_steps
    gen = torch.Generator(device="cpu").manual_seed(seed)
    noise = torch.randn(1, cfg.chunk_size, cfg.max_action_dim, generator=gen)
    cuda = device.type == "cuda"
    if cuda:
        torch.cuda.synchronize(device)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
    else:
        t0 = time.perf_counter()
    batch = {k: (v.to(device, non_blocking=True) if isinstance(v, torch.Tensor) else v) for k, v in batch_host.items()}
    with torch.inference_mode():
        actions = policy.sample_actions(batch, noise=noise.to(device))
    out = actions.float().cpu()
    if cuda:
        end.record()
        torch.cuda.synchronize(device)
        return out, start.elapsed_time(end) / 1e3
    return out, time.perf_counter() - t0


def main(argv=None) -> dict:
    args = parse_args(argv)
    action_dim = args.action_dim or DOMAIN_ACTION_DIM.get(args.domain)
    if action_dim is None:
        raise SystemExit(f"unknown --domain {args.domain!r}: give --action-dim, or one of {sorted(DOMAIN_ACTION_DIM)}")
    torch.manual_seed(args.seed)
    device = torch.device(args.device or ("cuda:0" if torch.cuda.is_available() else "cpu"))
    policy, cfg = build_policy(args, action_dim)
    policy.to(device)
    if device.type == "cuda":
        policy.to(torch.bfloat16)
    policy.eval()
    size = int(cfg.input_features["camera0"].shape[-1])
    image = load_image(args.image, size)
    batch_host = {"camera0": image, "state": torch.zeros(1, cfg.max_state_dim), "prompt": [args.prompt],
                  "img_is_pad": torch.zeros(1, 1, dtype=torch.bool)}
    if device.type == "cuda":
        batch_host = {k: (v.pin_memory() if isinstance(v, torch.Tensor) else v) for k, v in batch_host.items()}
    sweep = [int(s) for s in args.steps.split(",") if s.strip()] or [args.num_inference_steps]
    results, actions = [], None
    for n in sweep:
        if device.type == "cuda" and not args.no_graphs and hasattr(policy, "enable_cuda_graphs"):
            policy.enable_cuda_graphs(True)            # one capture per step count
        for _ in range(args.warmup):
            generate(policy, batch_host, device, n, args.seed)
        times = []
        for _ in range(max(1, args.repeats)):
            actions, dt = generate(policy, batch_host, device, n, args.seed)
            times.append(dt)
        latency = float(np.median(times))
        chunk = actions[0, :, :action_dim]
        print(f"[bench] steps={n:>3}  latency={latency:6.3f}s  action_shape={tuple(chunk.shape)}")
        results.append({"steps": n, "latency_s": latency, "finite": bool(torch.isfinite(chunk).all())})
    chunk = actions[0, :, :action_dim]
    payload = {"data": chunk.tolist(), "shape": list(chunk.shape), "dtype": "float32", "prompt": args.prompt,
               "domain": args.domain, "weights": args.checkpoint or "random initialisation", "device": str(device),
               "sweep": results}
    Path(args.output).parent.mkdir(parents=True, exist_ok=True)
    Path(args.output).write_text(json.dumps(payload))
    print("[summary] flow-matching steps -> action-generation latency:")
    for r in results:
        print(f"  {r['steps']:>3} steps  {r['latency_s'] * 1e3:9.2f} ms")
    return payload


if __name__ == "__main__":
    main()
