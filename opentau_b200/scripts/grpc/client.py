"""Client of the policy server, and the robot-side control loop that drives it
(reference ``src/opentau/scripts/grpc/client.py:60-601``).

:class:`PolicyClient` is transport only: requests with bounded retries, health as a plain dict, streaming.
:class:`RobotControlLoop` is the periodic robot-side step (latest joint state -> request -> one command), written
against two small callables so that it runs without a robot; :func:`make_ros2_node` binds it to ROS 2 topics when
``rclpy`` and the robot's message package are installed (they are not part of this framework's requirements).

    python -m opentau_b200.scripts.grpc.client --server_address 192.168.1.100:50051 --prompt "pick up the red block"
"""

from __future__ import annotations

import io
import logging
import time
import uuid
from dataclasses import dataclass, field
from typing import Callable

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


@dataclass
class ClientConfig:
    server_address: str = "127.0.0.1:50051"
    timeout_seconds: float = 5.0
    max_retries: int = 3
    retry_delay_seconds: float = 0.1
    image_encoding: str = "jpeg"          # jpeg | png | raw
    jpeg_quality: int = 85
    api_key: str | None = None
    max_message_mb: int = 100

    def __post_init__(self):
        if self.max_retries < 1:
            raise ValueError(f"max_retries must be at least 1, got {self.max_retries}")
        if self.image_encoding not in ("jpeg", "jpg", "png", "raw"):
            raise ValueError(f"image_encoding must be jpeg, png or raw, got {self.image_encoding!r}")


class PolicyClient:
    def __init__(self, address: str | ClientConfig = "127.0.0.1:50051", api_key: str | None = None,
                 max_message_mb: int = 100):
        self.config = address if isinstance(address, ClientConfig) else ClientConfig(
            server_address=address, api_key=api_key, max_message_mb=max_message_mb, timeout_seconds=30.0, max_retries=1)
        self.channel = self.stub = None
        self._requests = 0
        self.connect()

    def connect(self, wait_ready_s: float | None = None) -> bool:
        """Opens the channel (keep-alive pings, message limits); with ``wait_ready_s`` also waits that long for the
        server to answer and reports whether it did."""
        c = self.config
        opts = [("grpc.max_send_message_length", c.max_message_mb << 20),
                ("grpc.max_receive_message_length", c.max_message_mb << 20),
                ("grpc.keepalive_time_ms", 10000), ("grpc.keepalive_timeout_ms", 5000)]
        ch = grpc.insecure_channel(c.server_address, options=opts)
        if wait_ready_s is not None:
            try:
                grpc.channel_ready_future(ch).result(timeout=wait_ready_s)
            except grpc.FutureTimeoutError:
                ch.close()
                logging.error("no policy server answered at %s within %.1f s", c.server_address, wait_ready_s)
                return False
        if c.api_key:
            ch = grpc.intercept_channel(ch, ApiKeyClientInterceptor(c.api_key))
        self.channel, self.stub = ch, pb_grpc.RobotPolicyServiceStub(ch)
        return True

    def is_connected(self) -> bool:
        return self.stub is not None

    def disconnect(self) -> None:
        if self.channel is not None:
            self.channel.close()
        self.channel = self.stub = None

    def health(self, timeout: float = 5.0):
        return self.stub.HealthCheck(pb.HealthCheckRequest(), timeout=timeout)

    def health_check(self) -> dict:
        """Server health as a dict; an unreachable server is ``{"healthy": False, "status": <why>}``, not an error."""
        if self.stub is None:
            return {"healthy": False, "status": "not connected"}
        try:
            r = self.health(self.config.timeout_seconds)
        except grpc.RpcError as e:
            return {"healthy": False, "status": str(e)}
        return {"healthy": r.healthy, "status": r.status, "model_name": r.model_name, "device": r.device,
                "gpu_memory_used_gb": r.gpu_memory_used_gb, "gpu_memory_total_gb": r.gpu_memory_total_gb}

    def request_action_chunk(self, images: list[np.ndarray], state, prompt: str, prefix_action=None,
                             delay: int = 0) -> tuple[np.ndarray, float]:
        """``(chunk (T, D), server inference time in ms)`` with the configured encoding, time-out and retries; a chunk
        without steps comes back as an empty array.  ``RuntimeError`` after the last failed attempt."""
        if not self.is_connected():
            raise RuntimeError("the client is not connected to a server")
        c = self.config
        self._requests += 1
        req = self.make_request(images, state, prompt, prefix_action, delay, c.image_encoding, c.jpeg_quality)
        req.request_id = f"req_{self._requests}"
        last = None
        for attempt in range(c.max_retries):
            try:
                resp = self.stub.GetActionChunk(req, timeout=c.timeout_seconds)
                rows = [np.asarray(v.values, np.float32) for v in resp.action_chunk]
                return (np.stack(rows) if rows else np.zeros((0,), np.float32)), resp.inference_time_ms
            except grpc.RpcError as e:
                last = e
                logging.warning("request failed (attempt %d of %d): %s", attempt + 1, c.max_retries, e)
                if attempt + 1 < c.max_retries:
                    time.sleep(c.retry_delay_seconds)
        raise RuntimeError(f"failed after {c.max_retries} attempts: {last}")

    def make_request(self, images: list[np.ndarray], state, prompt: str, prefix_action=None, delay: int = 0,
                     encoding: str = "jpeg", quality: int = 90):
        req = pb.ObservationRequest(prompt=prompt, delay=delay, timestamp_ns=time.time_ns(), request_id=uuid.uuid4().hex)
        for im in images:
            req.images.append(encode_image(im, encoding, quality))
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
        self.disconnect()


# ---------------------------------------------------------------------------------------------------------------------
# robot side
# ---------------------------------------------------------------------------------------------------------------------
MOTOR_COMMANDS_TOPIC = "/motor_command_controller/motor_commands"
JOINT_STATES_TOPIC = "/joint_states"
#: the example robot's joints, in command order
JOINT_NAMES: tuple[str, ...] = ("base_yaw_joint", "shoulder_pitch_joint", "shoulder_roll_joint", "elbow_flex_joint",
                                "wrist_roll_joint", "wrist_yaw_joint", "hip_pitch_joint", "hip_roll_joint", "knee_joint",
                                "ankle_pitch_joint", "ankle_roll_joint", "gripper_finger_joint")


@dataclass
class RobotLoopConfig:
    server_address: str = "127.0.0.1:50051"
    timeout_seconds: float = 30.0                 # the first request may include the server's warm-up
    state_topic: str = JOINT_STATES_TOPIC
    motor_commands_topic: str = MOTOR_COMMANDS_TOPIC
    control_frequency_hz: float = 10.0
    prompt: str = ""
    num_cameras: int = 2
    image_height: int = 224
    image_width: int = 224
    joint_names: tuple[str, ...] = field(default_factory=lambda: JOINT_NAMES)


class RobotControlLoop:
    """One control period: latest joint state -> observation -> action chunk -> one joint command.

    ``publish(joint_names, positions)`` is the command sink; ``images()`` supplies the camera frames (default: fixed
    grey frames of the configured size, for robots whose cameras are not wired yet).  The state sent is positions
    followed by velocities of the first ``len(joint_names)`` joints.  The command applied is the LAST row of the chunk.
    Every way a period can end early (no server, no state yet, no prompt, a failed request, a malformed chunk) is
    reported through ``last_status`` and logged at most every 5 s; nothing is published then.  ``stop()`` publishes the
    current positions as the target (damping) before it disconnects."""

    def __init__(self, config: RobotLoopConfig, publish: Callable[[tuple[str, ...], list[float]], None],
                 client: PolicyClient | None = None, images: Callable[[], list[np.ndarray]] | None = None,
                 clock: Callable[[], float] = time.monotonic):
        self.config, self.publish, self.clock = config, publish, clock
        self.client = client or PolicyClient(ClientConfig(server_address=config.server_address,
                                                          timeout_seconds=config.timeout_seconds))
        self.images = images or self._fixed_images
        self.positions: list[float] | None = None
        self.velocities: list[float] | None = None
        self.last_status = "idle"
        self.last_inference_ms: float | None = None
        self._last_warned: dict[str, float] = {}

    def _fixed_images(self) -> list[np.ndarray]:
        c = self.config
        return [np.full((c.image_height, c.image_width, 3), 128, np.uint8) for _ in range(c.num_cameras)]

    def _warn(self, status: str, message: str) -> str:
        now = self.clock()
        if now - self._last_warned.get(status, -1e9) >= 5.0:
            self._last_warned[status] = now
            logging.warning(message)
        self.last_status = status
        return status

    def on_joint_state(self, positions, velocities) -> bool:
        """Keeps the first ``len(joint_names)`` joints of a state message; a shorter message is ignored."""
        n = len(self.config.joint_names)
        if len(positions) < n or len(velocities) < n:
            self._warn("short_state", f"joint state with fewer than {n} joints; waiting for a full one")
            return False
        self.positions, self.velocities = [float(x) for x in positions[:n]], [float(x) for x in velocities[:n]]
        return True

    def step(self) -> str:
        c = self.config
        if not self.client.is_connected():
            return self._warn("not_connected", "not connected to the policy server")
        if self.positions is None or self.velocities is None:
            return self._warn("no_state", "waiting for a joint state")
        if not c.prompt:
            return self._warn("no_prompt", "no prompt given")
        try:
            state = np.asarray(self.positions + self.velocities, np.float32)
            chunk, self.last_inference_ms = self.client.request_action_chunk(self.images(), state, c.prompt)
        except Exception as e:  # noqa: BLE001 - the loop outlives a failed period
            logging.error("no action chunk: %s", e)
            self.last_status = "request_failed"
            return self.last_status
        return self.apply(chunk)

    def apply(self, chunk: np.ndarray) -> str:
        n = len(self.config.joint_names)
        if chunk.ndim == 2:
            if chunk.shape[0] == 0:
                return self._warn("empty_chunk", "the action chunk has no steps")
            action = chunk[-1]
        elif chunk.ndim == 1 and chunk.shape[0] > 0:
            action = chunk
        else:
            return self._warn("bad_chunk", f"unexpected action chunk shape {chunk.shape}")
        if len(action) < n:
            return self._warn("short_action", f"the action has {len(action)} values, the robot {n} joints")
        self.publish(self.config.joint_names, [float(a) for a in action[:n]])
        self.last_status = "ok"
        return self.last_status

    def publish_damping_command(self) -> bool:
        if self.positions is None:
            return False
        self.publish(self.config.joint_names, list(self.positions))
        return True

    def stop(self) -> None:
        self.publish_damping_command()
        self.client.disconnect()


def make_ros2_node(config: RobotLoopConfig):
    """A ROS 2 node around :class:`RobotControlLoop`: subscribes to the joint states, publishes ``MotorCommands`` at the
    control frequency.  Needs ``rclpy``, ``sensor_msgs`` and the robot's ``interfaces`` message package."""
    try:
        import rclpy  # noqa: F401
        from interfaces.msg import MotorCommands, RawMotorCommand
        from rclpy.node import Node
        from sensor_msgs.msg import JointState
    except ImportError as e:
        raise ImportError(f"the ROS 2 client needs rclpy, sensor_msgs and the robot's message package ({e}); "
                          "RobotControlLoop itself runs without them") from e

    class PolicyNode(Node):
        def __init__(self):
            super().__init__("opentau_policy_client")
            self.pub = self.create_publisher(MotorCommands, config.motor_commands_topic, 10)
            self.loop = RobotControlLoop(config, self._publish)
            self.create_subscription(JointState, config.state_topic,
                                     lambda m: self.loop.on_joint_state(m.position, m.velocity), 10)
            self.create_timer(1.0 / config.control_frequency_hz, self.loop.step)

        def _publish(self, names, positions):
            msg = MotorCommands()
            msg.header.stamp = self.get_clock().now().to_msg()
            msg.joint_names = list(names)
            msg.commands = [RawMotorCommand(q=float(q)) for q in positions]
            self.pub.publish(msg)

        def destroy_node(self):
            self.loop.stop()
            super().destroy_node()

    return PolicyNode()


def main(argv: list[str] | None = None) -> None:
    import argparse
    ap = argparse.ArgumentParser(description="Robot-side client of the policy server (ROS 2).")
    ap.add_argument("--server_address", default="127.0.0.1:50051")
    ap.add_argument("--prompt", default="")
    ap.add_argument("--control_frequency", type=float, default=10.0)
    ap.add_argument("--num_cameras", type=int, default=2)
    ap.add_argument("--timeout", type=float, default=30.0)
    a = ap.parse_args(argv)
    cfg = RobotLoopConfig(server_address=a.server_address, prompt=a.prompt, control_frequency_hz=a.control_frequency,
                          num_cameras=a.num_cameras, timeout_seconds=a.timeout)
    import rclpy
    rclpy.init()
    node = make_ros2_node(cfg)
    try:
        rclpy.spin(node)
    except KeyboardInterrupt:
        pass
    finally:
        node.destroy_node()
        rclpy.shutdown()


if __name__ == "__main__":
    main()
