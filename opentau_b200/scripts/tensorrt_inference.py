"""Run the exported sampler through ONNX Runtime's TensorRT execution provider (reference
``src/opentau/scripts/tensorrt_inference.py:72-200``).

The engine is built on the first call (minutes for a 3 B-parameter graph) and cached beside the model, keyed by
precision, so later processes start in seconds; layers TensorRT cannot take fall back to the CUDA provider, then to
the CPU.  Pre- and post-processing and the timing loop are those of ``onnx_inference.py``.

    python -m opentau_b200.scripts.tensorrt_inference --checkpoint_dir outputs/export --n_repeats 20 [--no_fp16]
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

from .onnx_inference import OnnxInferenceArgs, benchmark


def tensorrt_provider_options(onnx_path: str | Path, cache_dir: str | Path | None = None, fp16: bool = True,
                              workspace_gb: int = 8) -> tuple[str, dict]:
    """The execution-provider entry for ``InferenceSession(providers=[...])``: engine + timing caches under
    ``<model>_trt_cache_<precision>``, half precision on request, a bounded builder workspace."""
    stem = Path(onnx_path).with_suffix("")
    cache = Path(cache_dir) if cache_dir else stem.parent / f"{stem.name}_trt_cache_{'fp16' if fp16 else 'fp32'}"
    cache.mkdir(parents=True, exist_ok=True)
    return ("TensorrtExecutionProvider", {
        "trt_engine_cache_enable": True, "trt_engine_cache_path": str(cache),
        "trt_timing_cache_enable": True, "trt_timing_cache_path": str(cache),
        "trt_fp16_enable": bool(fp16), "trt_max_workspace_size": int(workspace_gb) << 30})


def load_tensorrt_session(onnx_path: str | Path, cache_dir: str | Path | None = None, fp16: bool = True,
                          workspace_gb: int = 8, ort=None):
    """``ort``: the onnxruntime module (injected by tests; imported when None)."""
    if ort is None:
        try:
            import onnxruntime as ort
        except ImportError as e:
            raise RuntimeError("onnxruntime (with the TensorRT execution provider) is not installed") from e
    if not Path(onnx_path).is_file():
        raise FileNotFoundError(f"ONNX model not found: {onnx_path}")
    if "TensorrtExecutionProvider" not in ort.get_available_providers():
        raise RuntimeError("this onnxruntime build has no TensorRT execution provider; available: "
                           f"{ort.get_available_providers()}")
    trt = tensorrt_provider_options(onnx_path, cache_dir, fp16, workspace_gb)
    return ort.InferenceSession(str(onnx_path), providers=[trt, "CUDAExecutionProvider", "CPUExecutionProvider"])


def main(argv=None) -> dict:
    from ..utils.tokenizer import load_text_tokenizer
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--checkpoint_dir", default="outputs/export")
    ap.add_argument("--n_repeats", type=int, default=10)
    ap.add_argument("--num_cams", type=int, default=1)
    ap.add_argument("--prompt_max_length", type=int, default=256)
    ap.add_argument("--no_fp16", action="store_true")
    ap.add_argument("--workspace_gb", type=int, default=8)
    ap.add_argument("--cache_dir", default=None)
    a = ap.parse_args(argv)
    args = OnnxInferenceArgs(checkpoint_dir=a.checkpoint_dir, n_repeats=a.n_repeats, num_cams=a.num_cams,
                             prompt_max_length=a.prompt_max_length)
    session = load_tensorrt_session(Path(a.checkpoint_dir) / "model.onnx", a.cache_dir, not a.no_fp16, a.workspace_gb)
    summary = benchmark(session, load_text_tokenizer(args.tokenizer_path, args.vocab_size), args)
    print(json.dumps(summary))
    return summary


if __name__ == "__main__":
    main()
