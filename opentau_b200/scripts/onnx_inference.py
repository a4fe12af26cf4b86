"""Run an exported pi0.5 graph with ONNX Runtime (reference ``src/opentau/scripts/onnx_inference.py:127-300``).
Tokenisation and state discretisation happen here, outside the graph."""

from __future__ import annotations

import numpy as np


def load_session(path: str, providers: list[str] | None = None):
    try:
        import onnxruntime as ort
    except ImportError as e:
        raise RuntimeError("onnxruntime is not installed") from e
    return ort.InferenceSession(path, providers=providers or ["CUDAExecutionProvider", "CPUExecutionProvider"])


def run_inference(session, lang_tokens: np.ndarray, lang_masks: np.ndarray, images: list[np.ndarray], chunk: int,
                  max_action_dim: int, action_prefix: np.ndarray | None = None, delay: int = 0, seed: int | None = None):
    rng = np.random.default_rng(seed)
    B = lang_tokens.shape[0]
    feed = {"lang_tokens": lang_tokens.astype(np.int64), "lang_masks": lang_masks.astype(bool),
            "noise": rng.standard_normal((B, chunk, max_action_dim)).astype(np.float32),
            "action_prefix": (action_prefix if action_prefix is not None else np.zeros((B, chunk, max_action_dim))).astype(np.float32),
            "delay": np.array([delay], np.int64)}
    feed.update({f"image{i}": im.astype(np.float32) for i, im in enumerate(images)})
    return session.run(["actions"], feed)[0]
