"""``opentau-export``: export the pi0.5 sampler as one traceable graph (reference
``src/opentau/scripts/export_to_onnx.py:62-330``).

:class:`PI05OnnxWrapper` is the deployment-shaped module: it takes pre-tokenised language tokens, the initial noise,
the real-time-chunking prefix / delay and the camera images, and returns the un-normalised action chunk — every
non-tensor step (tokenisation, state discretisation) stays outside.  Tracing runs with the plain-PyTorch operator set
(the hand-written sm_100a kernels are opaque to a tracer and pointless on another runtime).  ``torch.onnx.export``
needs the ``onnx`` package; without it the wrapper can still be checked and saved with ``torch.export`` /
``torch.jit.trace`` (``--format torchscript``).
"""

from __future__ import annotations

import argparse
import logging
import os
from pathlib import Path

import torch
from torch import Tensor

from ..configs import parser
from ..configs.train import TrainPipelineConfig


class PI05OnnxWrapper(torch.nn.Module):
    def __init__(self, policy):
        super().__init__()
        self.policy = policy

    def forward(self, lang_tokens: Tensor, lang_masks: Tensor, noise: Tensor, action_prefix: Tensor, delay: Tensor,
                *images: Tensor) -> Tensor:
        pol = self.policy
        cfg = pol.config
        B = lang_tokens.shape[0]
        imgs = [im * 2.0 - 1.0 for im in images]
        masks = [torch.ones(B, dtype=torch.bool, device=lang_tokens.device) for _ in imgs]
        actions = pol.model.sample_actions(imgs, masks, lang_tokens, lang_masks.bool(), action_prefix=action_prefix,
                                           delay=delay, noise=noise)
        idx = torch.zeros(B, dtype=torch.long, device=actions.device)
        feat = cfg.action_feature
        real = feat.shape[0] if feat is not None else actions.shape[-1]
        return pol.unnormalize_outputs({"actions": actions[:, :, :real]}, idx)["actions"]


def example_inputs(policy, num_cams: int, device="cpu"):
    cfg = policy.config
    H, W = cfg.resize_imgs_with_padding
    B = 1
    return (torch.randint(3, 100, (B, cfg.prompt_max_length), device=device),
            torch.ones(B, cfg.prompt_max_length, dtype=torch.bool, device=device),
            torch.randn(B, cfg.chunk_size, cfg.max_action_dim, device=device),
            torch.zeros(B, cfg.chunk_size, cfg.max_action_dim, device=device),
            torch.zeros(1, dtype=torch.long, device=device),
            *[torch.rand(B, 3, H, W, device=device) for _ in range(num_cams)])


def export(policy, out_path: str | Path, num_cams: int = 1, fmt: str = "onnx", opset: int = 18) -> Path:
    prev = os.environ.get("OPENTAU_B200_ORACLE")
    os.environ["OPENTAU_B200_ORACLE"] = "1"            # trace the plain-PyTorch operator set
    try:
        wrapper = PI05OnnxWrapper(policy.float().eval().cpu())
        args = example_inputs(policy, num_cams)
        out_path = Path(out_path)
        out_path.parent.mkdir(parents=True, exist_ok=True)
        with torch.no_grad():
            if fmt == "onnx":
                try:
                    import onnx  # noqa: F401
                except ImportError as e:
                    raise RuntimeError("ONNX export needs the `onnx` package, which is not installed; use "
                                       "--format torchscript, or install onnx where the export runs") from e
                names = ["lang_tokens", "lang_masks", "noise", "action_prefix", "delay"] + [f"image{i}" for i in range(num_cams)]
                torch.onnx.export(wrapper, args, str(out_path), input_names=names, output_names=["actions"],
                                  opset_version=opset, do_constant_folding=True)
            elif fmt == "torchscript":
                traced = torch.jit.trace(wrapper, args, check_trace=False, strict=False)
                traced.save(str(out_path))
            else:
                raise ValueError(f"unknown export format {fmt!r}")
    finally:
        if prev is None:
            os.environ.pop("OPENTAU_B200_ORACLE", None)
        else:
            os.environ["OPENTAU_B200_ORACLE"] = prev
    return out_path


def main() -> None:
    from ..policies.factory import make_policy
    from ..utils.logging_utils import init_logging
    init_logging()
    ap = argparse.ArgumentParser(add_help=False)
    ap.add_argument("--output", default="outputs/export/policy.onnx")
    ap.add_argument("--format", default="onnx", choices=["onnx", "torchscript"])
    a, rest = ap.parse_known_args()
    cfg: TrainPipelineConfig = parser.parse_config(TrainPipelineConfig, rest)
    from ..policies.candidates import refuse_candidates
    refuse_candidates(cfg, reason="the exported graph is one sampler call at a static batch; candidates are expanded "
                      "and scored in the policy wrapper, outside of what is traced. Export with policy.n_candidates=1.")
    policy = make_policy(cfg.policy)
    out = export(policy, a.output, cfg.num_cams, a.format)
    logging.info("exported %s (%.1f MB)", out, out.stat().st_size / 1e6)


if __name__ == "__main__":
    main()
