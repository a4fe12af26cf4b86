"""Client of the policy server (the reference client ``src/opentau/scripts/grpc/client.py:60-601`` is a ROS 2 node;
this one is transport only, so a ROS node, a teleoperation loop or a test can drive it)."""

from __future__ import annotations

import io
import time
import uuid

import grpc
import numpy as np

from . import robot_inference_pb2 as pb
from . import robot_inference_pb2_grpc as pb_grpc
from .auth import ApiKeyClientInterceptor


def encode_image(img: np.ndarray, encoding: str = "jpeg", quality: int = 90) -> "pb.CameraImage":
    """``(H,W,3)`` uint8 RGB -> message."""
    if encoding == "raw":
        h, w = img.shape[:2]
        return pb.CameraImage(image_data=np.ascontiguousarray(img, np.uint8).tobytes(), encoding=f"raw:{h}x{w}")
    from PIL import Image
    buf = io.BytesIO()
    Image.fromarray(img).save(buf, format="JPEG" if encoding in ("jpeg", "jpg") else "PNG", quality=quality)
    return pb.CameraImage(image_data=buf.getvalue(), encoding=encoding)


class PolicyClient:
    def __init__(self, address: str = "127.0.0.1:50051", api_key: str | None = None, max_message_mb: int = 100):
        opts = [("grpc.max_send_message_length", max_message_mb << 20),
                ("grpc.max_receive_message_length", max_message_mb << 20)]
        ch = grpc.insecure_channel(address, options=opts)
        if api_key:
            ch = grpc.intercept_channel(ch, ApiKeyClientInterceptor(api_key))
        self.channel = ch
        self.stub = pb_grpc.RobotPolicyServiceStub(ch)

    def health(self, timeout: float = 5.0):
        return self.stub.HealthCheck(pb.HealthCheckRequest(), timeout=timeout)

    def make_request(self, images: list[np.ndarray], state, prompt: str, prefix_action=None, delay: int = 0,
                     encoding: str = "jpeg"):
        req = pb.ObservationRequest(prompt=prompt, delay=delay, timestamp_ns=time.time_ns(), request_id=uuid.uuid4().hex)
        for im in images:
            req.images.append(encode_image(im, encoding))
        req.robot_state.state.extend([float(x) for x in np.asarray(state).reshape(-1)])
        if prefix_action is not None:
            for row in np.asarray(prefix_action):
                req.prefix_action.add(values=[float(x) for x in row])
        return req

    def get_action_chunk(self, images, state, prompt, prefix_action=None, delay: int = 0, encoding: str = "jpeg",
                         timeout: float = 30.0) -> tuple[np.ndarray, "pb.ActionChunkResponse"]:
        resp = self.stub.GetActionChunk(self.make_request(images, state, prompt, prefix_action, delay, encoding),
                                        timeout=timeout)
        return np.asarray([list(v.values) for v in resp.action_chunk], np.float32), resp

    def stream(self, requests):
        for resp in self.stub.StreamActionChunks(iter(requests)):
            yield np.asarray([list(v.values) for v in resp.action_chunk], np.float32), resp

    def close(self) -> None:
        self.channel.close()
