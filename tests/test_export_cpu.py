"""The export wrapper is one traceable function of tensors and reproduces the policy's sampler."""

import pytest
import torch

from helpers import tiny_batch, tiny_pi05
from opentau_b200.scripts.export_to_onnx import PI05OnnxWrapper, example_inputs, export


def test_wrapper_matches_policy_and_traces(tmp_path):
    pol = tiny_pi05(num_steps=2, prompt_max_length=16).eval()
    b = tiny_batch(batch_size=1)
    noise = torch.randn(1, 10, 32)
    want = pol.sample_actions(b, noise=noise)
    w = PI05OnnxWrapper(pol)
    got = w(b["lang_tokens"], b["lang_masks"], noise, torch.zeros(1, 10, 32), torch.zeros(1, dtype=torch.long), b["camera0"])
    assert torch.allclose(got, want, atol=1e-5)
    path = export(pol, tmp_path / "p.pt", num_cams=1, fmt="torchscript")
    mod = torch.jit.load(str(path))
    args = example_inputs(pol, 1)
    assert torch.allclose(mod(*args), w(*args), atol=1e-4)
    import os
    assert "OPENTAU_B200_ORACLE" not in os.environ
    try:
        import onnx  # noqa: F401
    except ImportError:
        with pytest.raises(RuntimeError, match="onnx"):
            export(pol, tmp_path / "p.onnx", fmt="onnx")
    assert "OPENTAU_B200_ORACLE" not in os.environ
