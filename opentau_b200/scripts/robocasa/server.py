"""Websocket policy server for RoboCasa clients (reference ``src/opentau/scripts/robocasa/server.py:96-652``).

Wire format (MessagePack over websocket): a request is ``{"images": {camera: jpeg bytes}, "state": [..],
"prompt": str}`` or ``{"batch": true, "items": [request, ...]}``; the reply is the action chunk as nested lists
``(T, action_dim)`` (a list of chunks for a batch).  With ``"include_accel": true`` the reply is
``{"actions": ..., "accel": ...}``.  A failed step answers with a zero chunk so the simulator's control loop keeps
its cadence.  All environments of a batch request go through ONE ``sample_actions`` call.
"""

from __future__ import annotations

import asyncio
import io
import logging
from typing import Any

import msgpack
import numpy as np
import torch

from ...configs import parser
from ...configs.train import TrainPipelineConfig

logger = logging.getLogger(__name__)

ROBOCASA_HOST = "0.0.0.0"  # nosec B104 - default listen address; restrict with --robocasa_host
ROBOCASA_PORT = 8765
ROBOCASA_ACTION_DIM = 16
ROBOCASA_CAMERA_ORDER = ("robot0_eye_in_hand", "robot0_agentview_left", "robot0_agentview_right")
_ERROR_RESPONSE_CHUNK_STEPS = 8


def jpeg_bytes_to_rgb(jpeg_bytes: bytes) -> np.ndarray:
    from PIL import Image
    return np.asarray(Image.open(io.BytesIO(jpeg_bytes)).convert("RGB"))


def decode_all_images(images: dict[str, bytes]) -> dict[str, np.ndarray]:
    return {k: jpeg_bytes_to_rgb(v) for k, v in images.items()}


def unpack_payload_dict(data: dict) -> tuple[dict[str, bytes], np.ndarray, str]:
    images, state, prompt = data.get("images"), data.get("state"), data.get("prompt", "")
    if not isinstance(images, dict):
        raise ValueError("Expected 'images' dict")
    if not isinstance(state, list):
        raise ValueError("Expected 'state' list")
    images = {str(k): (v if isinstance(v, (bytes, bytearray)) else bytes(v)) for k, v in images.items()}
    return images, np.asarray(state, dtype=np.float64), str(prompt) if prompt is not None else ""


def pack_action(chunk: np.ndarray) -> bytes:
    a = np.asarray(chunk, dtype=np.float64)
    if a.ndim != 2:
        raise ValueError(f"Expected action chunk of shape (T, action_dim), got shape {a.shape}")
    return msgpack.packb(a.tolist(), use_bin_type=True)


def pack_actions_batch(chunks: list[np.ndarray]) -> bytes:
    return msgpack.packb([np.asarray(c, dtype=np.float64).tolist() for c in chunks], use_bin_type=True)


def pack_action_envelope(chunk: np.ndarray, accel: float | None) -> bytes:
    a = np.asarray(chunk, dtype=np.float64)
    if a.ndim != 2:
        raise ValueError(f"Expected action chunk of shape (T, action_dim), got shape {a.shape}")
    return msgpack.packb({"actions": a.tolist(), "accel": accel}, use_bin_type=True)


def pack_actions_batch_envelope(chunks: list[np.ndarray], accel: list[float] | None) -> bytes:
    return msgpack.packb({"actions": [np.asarray(c, dtype=np.float64).tolist() for c in chunks], "accel": accel},
                         use_bin_type=True)


def build_batch(cfg, items: list[tuple[dict[str, np.ndarray], np.ndarray, str]], device) -> dict[str, Any]:
    """Requests -> one policy batch: cameras in the fixed RoboCasa order (missing ones are flagged as padding)."""
    from ... import ops
    H, W = cfg.resolution
    B = len(items)
    batch: dict[str, Any] = {}
    pads = torch.zeros(B, cfg.num_cams, dtype=torch.bool)
    for ci in range(cfg.num_cams):
        name = ROBOCASA_CAMERA_ORDER[ci] if ci < len(ROBOCASA_CAMERA_ORDER) else f"camera{ci}"
        frames = []
        for bi, (imgs, _, _) in enumerate(items):
            arr = imgs.get(name)
            if arr is None:
                pads[bi, ci] = True
                frames.append(torch.zeros(3, H, W))
                continue
            t = torch.from_numpy(np.ascontiguousarray(arr)).permute(2, 0, 1)[None].float() / 255.0
            if tuple(t.shape[-2:]) != (H, W):
                t = ops.resize_with_pad(t, W, H, pad_value=0.0)
            frames.append(t[0])
        batch[f"camera{ci}"] = torch.stack(frames).to(device)
    state = torch.zeros(B, cfg.max_state_dim)
    for bi, (_, st, _) in enumerate(items):
        n = min(len(st), cfg.max_state_dim)
        state[bi, :n] = torch.from_numpy(st[:n]).float()
    batch["state"] = state.to(device)
    batch["prompt"] = [p for _, _, p in items]
    batch["img_is_pad"] = pads.to(device)
    return batch


class OpenTauRoboCasaPolicy:
    def __init__(self, cfg: TrainPipelineConfig, policy=None, accel_prefix: int | str | None = None):
        from ...policies.accel import configure_accel
        from ...policies.factory import make_policy
        from ...utils.utils import auto_torch_device
        self.cfg, self.device = cfg, auto_torch_device()
        self.policy = policy if policy is not None else make_policy(cfg.policy)
        self.policy.to(self.device)
        if self.device.type == "cuda":
            self.policy.to(torch.bfloat16)
        self.policy.eval()
        # precedence: this entry point's flag, then cfg.policy.accel_prefix, then $OPENTAU_ACCEL_PREFIX
        self.accel_prefix = configure_accel(self.policy, cfg, override=accel_prefix)
        from ...policies.candidates import configure_candidates
        self.n_candidates = configure_candidates(self.policy, cfg, device=self.device)
        self.last_accel: list[float] | None = None

    def infer_batch(self, items, action_dim: int) -> list[np.ndarray]:
        from ...configs.deployment import tag_norm_head
        batch = tag_norm_head(build_batch(self.cfg, items, self.device), getattr(self.cfg, "server", None))
        with torch.inference_mode():
            actions = self.policy.sample_actions(batch).float().cpu().numpy()
        acc = getattr(self.policy, "last_accel", None) if self.accel_prefix else None
        self.last_accel = list(acc) if acc is not None and len(acc) == len(items) else None
        return [a[:, :action_dim] for a in actions]

    def infer(self, images, state, prompt, action_dim: int) -> np.ndarray:
        return self.infer_batch([(images, state, prompt)], action_dim)[0]


def make_handler(action_dim: int, runner: OpenTauRoboCasaPolicy):
    async def handler(websocket: Any):
        async for message in websocket:
            data = None
            try:
                data = msgpack.unpackb(message, raw=False)
                if not isinstance(data, dict):
                    raise ValueError("Expected dict payload")
                want_accel = data.get("include_accel") is True
                if data.get("batch") is True:
                    items = data.get("items")
                    if not isinstance(items, list):
                        raise ValueError("Batch request requires 'items' list")
                    decoded = []
                    for it in items:
                        imgs, st, prompt = unpack_payload_dict(it)
                        decoded.append((decode_all_images(imgs), st, prompt))
                    out = await asyncio.to_thread(runner.infer_batch, decoded, action_dim)
                    await websocket.send(pack_actions_batch_envelope(out, runner.last_accel) if want_accel
                                         else pack_actions_batch(out))
                else:
                    imgs, st, prompt = unpack_payload_dict(data)
                    act = await asyncio.to_thread(runner.infer, decode_all_images(imgs), st, prompt, action_dim)
                    acc = runner.last_accel[0] if runner.last_accel else None
                    await websocket.send(pack_action_envelope(act, acc) if want_accel else pack_action(act))
            except Exception as e:  # noqa: BLE001 - the simulator must get an answer
                logger.exception("Policy step failed: %s", e)
                zero = [[0.0] * action_dim for _ in range(_ERROR_RESPONSE_CHUNK_STEPS)]
                is_batch = isinstance(data, dict) and data.get("batch") is True
                want_accel = isinstance(data, dict) and data.get("include_accel") is True
                n = len(data.get("items") or []) if is_batch else 0
                payload: Any = [zero for _ in range(n)] if is_batch else zero
                if want_accel:
                    payload = {"actions": payload, "accel": None}
                await websocket.send(msgpack.packb(payload, use_bin_type=True))
    return handler


async def serve(cfg: TrainPipelineConfig, runner: OpenTauRoboCasaPolicy | None = None, host: str = ROBOCASA_HOST,
                port: int = ROBOCASA_PORT, action_dim: int = ROBOCASA_ACTION_DIM, ready: asyncio.Event | None = None,
                stop: asyncio.Event | None = None):
    import websockets
    runner = runner or OpenTauRoboCasaPolicy(cfg)
    async with websockets.serve(make_handler(action_dim, runner), host, port, max_size=None) as server:
        if ready is not None:
            ready.port = server.sockets[0].getsockname()[1]  # type: ignore[attr-defined]
            ready.set()
        logger.info("RoboCasa policy server on ws://%s:%d", host, port)
        await (stop.wait() if stop is not None else asyncio.Future())


@parser.wrap()
def main(cfg: TrainPipelineConfig):
    from ...utils.logging_utils import init_logging
    init_logging()
    asyncio.run(serve(cfg))


if __name__ == "__main__":
    main()
