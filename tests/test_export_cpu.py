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


def test_runner_prepares_the_feed_and_drives_an_exported_graph(tmp_path):
    """``onnx_inference.run_inference`` in front of the TorchScript export: state discretisation into the prompt,
    tokenisation to the exported length, shape checks, the feed's names and dtypes, the timing summary; the TensorRT
    loader builds its provider options and refuses a runtime without that provider."""
    import numpy as np
    from opentau_b200.scripts import onnx_inference as oi
    from opentau_b200.scripts.tensorrt_inference import load_tensorrt_session, tensorrt_provider_options
    from opentau_b200.utils.tokenizer import HashTokenizer
    assert oi.prepare_discrete_state(np.array([[-1.0, 0.0, 1.0, 5.0]])) == ["0 128 255 255"]
    assert oi.build_prompt("lift", "1 2") == "Task: lift, State: 1 2;\n"
    pol = tiny_pi05(num_steps=2, prompt_max_length=16).eval()
    export(pol, tmp_path / "policy.pt", num_cams=1, fmt="torchscript")
    args = oi.OnnxInferenceArgs(checkpoint_dir=str(tmp_path), n_action_steps=10, prompt_max_length=16, num_cams=1,
                                vocab_size=1024, n_repeats=2, dump_path=str(tmp_path / "dump.pkl"))
    tok = HashTokenizer(1024)
    sess = oi.TorchScriptSession(tmp_path / "policy.pt")

    class Spy:
        def __init__(self, inner):
            self.inner, self.feeds = inner, []

        def run(self, names, feed):
            self.feeds.append(feed)
            return self.inner.run(names, feed)
    spy = Spy(sess)
    state = np.zeros((1, 32), np.float32)
    img = np.random.default_rng(0).uniform(0, 1, (1, 3, 224, 224)).astype(np.float32)
    noise = np.random.default_rng(1).standard_normal((1, 10, 32)).astype(np.float32)
    out = oi.run_inference(spy, tok, args, prompt="lift the cup", state=state, images=[img], noise=noise)
    feed = spy.feeds[0]
    assert set(feed) == {"lang_tokens", "lang_masks", "noise", "action_prefix", "delay", "image0"}
    assert feed["lang_tokens"].shape == (1, 16) and feed["lang_tokens"].dtype == np.int64
    assert feed["lang_masks"].dtype == bool and feed["delay"].tolist() == [0] and not feed["action_prefix"].any()
    assert out.shape[:2] == (1, 10) and np.isfinite(out).all()
    again = oi.run_inference(spy, tok, args, prompt="lift the cup", state=state, images=[img], noise=noise)
    assert np.allclose(out, again)                                   # same noise, same chunk
    with pytest.raises(ValueError, match="num_cams"):
        oi.run_inference(spy, tok, args, prompt="x", state=state, images=[img, img])
    with pytest.raises(ValueError, match="expected"):
        oi.run_inference(spy, tok, args, prompt="x", state=state, images=[img[:, :, :100]])
    with pytest.raises(ValueError, match="delay"):
        oi.run_inference(spy, tok, args, prompt="x", state=state, images=[img], delay=11)
    summary = oi.benchmark(spy, tok, args)
    assert summary["n"] == 1 and summary["finite"] and (tmp_path / "dump.pkl").exists()
    name, opts = tensorrt_provider_options(tmp_path / "model.onnx", fp16=False)
    assert name == "TensorrtExecutionProvider" and opts["trt_fp16_enable"] is False
    assert opts["trt_engine_cache_path"].endswith("model_trt_cache_fp32")
    (tmp_path / "model.onnx").write_bytes(b"x")

    class FakeOrt:
        @staticmethod
        def get_available_providers():
            return ["CPUExecutionProvider"]
    with pytest.raises(RuntimeError, match="no TensorRT execution provider"):
        load_tensorrt_session(tmp_path / "model.onnx", ort=FakeOrt)
