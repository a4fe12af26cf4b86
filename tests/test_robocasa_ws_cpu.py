"""RoboCasa websocket policy server on the loopback interface: single and batched requests, accel envelope, and the
zero-chunk answer to a malformed request."""

import asyncio
import io

import msgpack
import numpy as np
import pytest

pytest.importorskip("websockets")

from helpers import tiny_pi05  # noqa: E402
from opentau_b200.configs.train import TrainPipelineConfig  # noqa: E402
from opentau_b200.scripts.robocasa.server import OpenTauRoboCasaPolicy, ROBOCASA_CAMERA_ORDER, serve  # noqa: E402


def _jpeg(seed):
    from PIL import Image
    arr = np.random.default_rng(seed).integers(0, 255, (48, 64, 3), dtype=np.uint8)
    buf = io.BytesIO()
    Image.fromarray(arr).save(buf, format="JPEG")
    return buf.getvalue()


def test_single_batch_and_error_replies():
    import websockets
    pol = tiny_pi05(num_steps=2)
    cfg = TrainPipelineConfig.from_dict({"policy": {"type": "pi05"}, "resolution": [224, 224], "num_cams": 1,
                                         "action_chunk": 10, "batch_size": 1})
    cfg.policy = pol.config
    runner = OpenTauRoboCasaPolicy(cfg, policy=pol)

    async def run():
        ready, stop = asyncio.Event(), asyncio.Event()
        task = asyncio.create_task(serve(cfg, runner, host="127.0.0.1", port=0, action_dim=7, ready=ready, stop=stop))
        await ready.wait()
        req = {"images": {ROBOCASA_CAMERA_ORDER[0]: _jpeg(0)}, "state": [0.1] * 9, "prompt": "open the drawer"}
        async with websockets.connect(f"ws://127.0.0.1:{ready.port}", max_size=None) as ws:
            await ws.send(msgpack.packb(req, use_bin_type=True))
            one = msgpack.unpackb(await ws.recv(), raw=False)
            await ws.send(msgpack.packb({"batch": True, "include_accel": True, "items": [req, req]}, use_bin_type=True))
            two = msgpack.unpackb(await ws.recv(), raw=False)
            await ws.send(msgpack.packb({"images": "nope", "state": [0.0]}, use_bin_type=True))
            bad = msgpack.unpackb(await ws.recv(), raw=False)
        stop.set()
        await task
        return one, two, bad

    one, two, bad = asyncio.run(run())
    assert np.asarray(one).shape == (10, 7) and np.isfinite(np.asarray(one)).all()
    assert set(two) == {"actions", "accel"} and np.asarray(two["actions"]).shape == (2, 10, 7) and two["accel"] is None
    assert np.asarray(bad).shape == (8, 7) and not np.asarray(bad).any()
