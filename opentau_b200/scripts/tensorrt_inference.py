"""ONNX Runtime session with the TensorRT execution provider (reference
``src/opentau/scripts/tensorrt_inference.py:72-200``): engine cache next to the model, fp16 enabled, CUDA fallback."""

from __future__ import annotations

from pathlib import Path


def load_tensorrt_session(onnx_path: str, cache_dir: str | None = None, fp16: bool = True, workspace_gb: int = 8):
    try:
        import onnxruntime as ort
    except ImportError as e:
        raise RuntimeError("onnxruntime (with the TensorRT execution provider) is not installed") from e
    cache = Path(cache_dir or Path(onnx_path).with_suffix("").as_posix() + "_trt_cache")
    cache.mkdir(parents=True, exist_ok=True)
    trt = ("TensorrtExecutionProvider", {"trt_engine_cache_enable": True, "trt_engine_cache_path": str(cache),
                                         "trt_fp16_enable": fp16, "trt_max_workspace_size": workspace_gb << 30})
    if "TensorrtExecutionProvider" not in ort.get_available_providers():
        raise RuntimeError("this onnxruntime build has no TensorRT execution provider")
    return ort.InferenceSession(onnx_path, providers=[trt, "CUDAExecutionProvider", "CPUExecutionProvider"])
