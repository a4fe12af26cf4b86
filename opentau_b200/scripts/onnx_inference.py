"""Run an exported pi0.5 sampler graph outside the training framework (reference
``src/opentau/scripts/onnx_inference.py:60-300``).

Everything that is not a tensor operation happens here, in front of the graph: the state is discretised into 256 bins
and written into the prompt (``Task: <task>, State: <bins>;\\n``, the training-time format), the prompt is tokenised
and padded to ``prompt_max_length``, the initial noise and the real-time-chunking prefix / delay are prepared, the
camera images are checked against the exported resolution.  The graph itself is opaque: any object with
``run(output_names, feed) -> [actions]`` serves — an ONNX Runtime session (:func:`load_onnx_session`, needs the
``onnxruntime`` package), the TensorRT execution provider (``tensorrt_inference.py``), or
:class:`TorchScriptSession` around the ``--format torchscript`` export, which needs nothing but torch.

    python -m opentau_b200.scripts.onnx_inference --checkpoint_dir outputs/export --prompt "pick up the block" \\
        --n_repeats 20 [--provider CUDAExecutionProvider] [--torchscript]
"""

from __future__ import annotations

import argparse
import json
import pickle
import time
from dataclasses import dataclass
from pathlib import Path

import numpy as np


@dataclass
class OnnxInferenceArgs:
    """Shapes the graph was exported with, and the prompt settings of the policy."""
    checkpoint_dir: str = "outputs/export"
    prompt: str = "pick up the red block and place it in the bin"
    n_action_steps: int = 50
    max_action_dim: int = 32
    max_state_dim: int = 32
    prompt_max_length: int = 256
    num_cams: int = 1
    resolution_height: int = 224
    resolution_width: int = 224
    tokenizer_path: str = "google/paligemma-3b-pt-224"
    vocab_size: int = 257152
    predict_response: bool = False
    n_repeats: int = 10
    provider: str | None = None
    delay: int = 0
    seed: int | None = 0
    dump_path: str | None = None        # pickle of the first call's feed and output


def prepare_discrete_state(state: np.ndarray) -> list[str]:
    """``state (B, D)`` in [-1, 1] (clipped) -> one string of 256-bin indices per sample
    (the training-time discretisation, ``policies/pi05/modeling_pi05.py: prepare_discrete_state``)."""
    s = np.clip(np.asarray(state, np.float32), -1.0, 1.0)
    idx = np.clip(((s + 1.0) * 128.0).astype(np.int64), 0, 255)
    return [" ".join(map(str, row)) for row in idx]


def build_prompt(task: str, state_str: str) -> str:
    return f"Task: {task}, State: {state_str};\n"


def tokenize_prompts(tokenizer, prompts: list[str], max_length: int) -> tuple[np.ndarray, np.ndarray]:
    enc = tokenizer(prompts, padding="max_length", padding_side="right", max_length=max_length, return_tensors="pt",
                    truncation=True)
    return np.asarray(enc["input_ids"], np.int64), np.asarray(enc["attention_mask"]).astype(bool)


def load_onnx_session(checkpoint_dir: str | Path, provider: str | None = None):
    """``model.onnx`` (+ external weights beside it) as an ONNX Runtime session: the requested provider, else CUDA
    with a CPU fallback when the build has it, else CPU; all graph optimisations on."""
    try:
        import onnxruntime as ort
    except ImportError as e:
        raise RuntimeError("onnxruntime is not installed; run the TorchScript export with --torchscript instead") from e
    path = Path(checkpoint_dir) / "model.onnx"
    if not path.is_file():
        raise FileNotFoundError(f"ONNX model not found: {path}")
    if provider:
        providers = [provider]
    elif ort.get_device() == "GPU":
        providers = ["CUDAExecutionProvider", "CPUExecutionProvider"]
    else:
        providers = ["CPUExecutionProvider"]
    opts = ort.SessionOptions()
    opts.graph_optimization_level = ort.GraphOptimizationLevel.ORT_ENABLE_ALL
    return ort.InferenceSession(str(path), sess_options=opts, providers=providers)


class TorchScriptSession:
    """The ``run(output_names, feed)`` surface of an inference session around a traced sampler
    (``opentau-export --format torchscript``)."""

    def __init__(self, path: str | Path, device: str = "cpu"):
        import torch
        self.torch, self.device = torch, device
        self.module = torch.jit.load(str(path), map_location=device).eval()

    def run(self, output_names, feed: dict[str, np.ndarray]) -> list[np.ndarray]:
        t = self.torch
        order = ["lang_tokens", "lang_masks", "noise", "action_prefix", "delay"]
        images = sorted((k for k in feed if k.startswith("image")), key=lambda k: int(k[5:]))
        args = [t.from_numpy(np.ascontiguousarray(feed[k])).to(self.device) for k in order + images]
        with t.no_grad():
            return [self.module(*args).float().cpu().numpy()]


def run_inference(session, tokenizer, args: OnnxInferenceArgs, *, prompt: str, state: np.ndarray,
                  images: list[np.ndarray], noise: np.ndarray | None = None, action_prefix: np.ndarray | None = None,
                  delay: int = 0, rng: np.random.Generator | None = None, dump_path: str | Path | None = None) -> np.ndarray:
    """One action chunk ``(B, n_action_steps, action_dim)`` in the robot's units.  ``state (B, max_state_dim)`` in
    [-1, 1]; ``images``: ``num_cams`` arrays ``(B, 3, H, W)`` in [0, 1] at the exported resolution; ``action_prefix``
    + ``delay``: the already committed first ``delay`` steps of the chunk (real-time chunking), zeros when absent."""
    state = np.asarray(state, np.float32)
    if state.ndim != 2:
        raise ValueError(f"state must be (batch, state_dim), got {state.shape}")
    B = state.shape[0]
    rng = rng or np.random.default_rng()
    prompts = [build_prompt(prompt, s) for s in prepare_discrete_state(state)]
    lang_tokens, lang_masks = tokenize_prompts(tokenizer, prompts, args.prompt_max_length)
    shape = (B, args.n_action_steps, args.max_action_dim)
    noise = rng.standard_normal(shape, dtype=np.float32) if noise is None else np.asarray(noise, np.float32)
    if noise.shape != shape:
        raise ValueError(f"noise shape {noise.shape} != {shape}")
    action_prefix = np.zeros(shape, np.float32) if action_prefix is None else np.asarray(action_prefix, np.float32)
    if action_prefix.shape != shape:
        raise ValueError(f"action_prefix shape {action_prefix.shape} != {shape}")
    if not 0 <= int(delay) <= args.n_action_steps:
        raise ValueError(f"delay {delay} outside [0, {args.n_action_steps}]")
    if len(images) != args.num_cams:
        raise ValueError(f"expected {args.num_cams} images (num_cams), got {len(images)}")
    res = (args.resolution_height, args.resolution_width)
    for i, im in enumerate(images):
        if im.ndim != 4 or im.shape[1] != 3 or tuple(im.shape[2:]) != res:
            raise ValueError(f"image {i} has shape {im.shape}: expected (batch, 3, {res[0]}, {res[1]})")
        if im.shape[0] != B:
            raise ValueError(f"image {i} batch size {im.shape[0]} != state batch size {B}")
    feed = {"lang_tokens": lang_tokens, "lang_masks": lang_masks, "noise": noise, "action_prefix": action_prefix,
            "delay": np.array([int(delay)], np.int64)}
    feed.update({f"image{i}": np.asarray(im, np.float32) for i, im in enumerate(images)})
    actions = session.run(["actions"], feed)[0]
    if dump_path is not None:
        with open(dump_path, "wb") as f:
            pickle.dump({"feed": feed, "actions": actions}, f)
    return actions


def benchmark(session, tokenizer, args: OnnxInferenceArgs) -> dict:
    """``n_repeats`` calls on a random observation (the first one is reported apart: it carries engine building /
    lazy initialisation); returns the timing summary that ``main`` prints."""
    rng = np.random.default_rng(args.seed)
    state = rng.uniform(-1, 1, (1, args.max_state_dim)).astype(np.float32)
    images = [rng.uniform(0, 1, (1, 3, args.resolution_height, args.resolution_width)).astype(np.float32)
              for _ in range(args.num_cams)]
    times, out = [], None
    for i in range(max(1, args.n_repeats)):
        t0 = time.perf_counter()
        out = run_inference(session, tokenizer, args, prompt=args.prompt, state=state, images=images, delay=args.delay,
                            rng=rng, dump_path=args.dump_path if i == 0 else None)
        times.append((time.perf_counter() - t0) * 1e3)
    rest = times[1:] or times
    return {"first_call_ms": times[0], "mean_ms": float(np.mean(rest)), "p50_ms": float(np.median(rest)),
            "max_ms": float(np.max(rest)), "n": len(rest), "actions_shape": list(out.shape),
            "finite": bool(np.isfinite(out).all())}


def parse_args(argv=None) -> tuple[OnnxInferenceArgs, bool]:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    for name, field in OnnxInferenceArgs.__dataclass_fields__.items():
        t = field.type if isinstance(field.type, type) else str
        if field.default is False:
            ap.add_argument(f"--{name}", action="store_true")
        else:
            ap.add_argument(f"--{name}", default=field.default,
                            type=(int if isinstance(field.default, int) and not isinstance(field.default, bool) else str))
    ap.add_argument("--torchscript", action="store_true", help="run policy.pt (the TorchScript export) instead of model.onnx")
    ns = vars(ap.parse_args(argv))
    ts = ns.pop("torchscript")
    for k in ("seed", "delay"):
        ns[k] = None if ns[k] in (None, "None") else int(ns[k])
    return OnnxInferenceArgs(**ns), ts


def main(argv=None) -> dict:
    from ..utils.tokenizer import load_text_tokenizer
    args, torchscript = parse_args(argv)
    tok = load_text_tokenizer(args.tokenizer_path, args.vocab_size)
    if torchscript:
        session = TorchScriptSession(Path(args.checkpoint_dir) / "policy.pt")
    else:
        session = load_onnx_session(args.checkpoint_dir, args.provider)
    summary = benchmark(session, tok, args)
    print(json.dumps(summary))
    return summary


if __name__ == "__main__":
    main()
