"""gRPC policy server: ``GetActionChunk``, ``StreamActionChunks``, ``HealthCheck``.

Behaviour of the reference server (``src/opentau/scripts/grpc/server.py:93-690``): decode the camera images (JPEG /
PNG / raw), resize-with-pad to the pipeline resolution, pad the state, run ``policy.sample_actions`` and return the
un-normalised chunk with the inference time; optional API-key interceptor; health check with GPU memory.  All
device work happens on ONE dedicated inference thread: request threads hand over a closure and wait, so the CUDA
graph captured for the sampler is always replayed from the thread (and stream) that captured it.
"""

from __future__ import annotations

import io
import logging
import queue
import threading
import time
from concurrent import futures
from typing import Any, Iterator

import grpc
import numpy as np
import torch

from ...configs import parser
from ...configs.train import TrainPipelineConfig
from . import robot_inference_pb2 as pb
from . import robot_inference_pb2_grpc as pb_grpc
from .auth import ApiKeyInterceptor, load_api_keys

logger = logging.getLogger(__name__)


class InferenceThread:
    """Runs submitted callables one at a time on a single long-lived thread."""

    def __init__(self, name: str = "policy-infer"):
        self.q: queue.Queue = queue.Queue()
        self.thread = threading.Thread(target=self._run, name=name, daemon=True)
        self.thread.start()

    def _run(self) -> None:
        while True:
            item = self.q.get()
            if item is None:
                return
            fn, fut = item
            try:
                fut.set_result(fn())
            except BaseException as e:  # noqa: BLE001 - delivered to the caller
                fut.set_exception(e)

    def submit(self, fn) -> futures.Future:
        fut: futures.Future = futures.Future()
        self.q.put((fn, fut))
        return fut

    def stop(self) -> None:
        self.q.put(None)
        self.thread.join(timeout=5)


def decode_image(img: "pb.CameraImage") -> np.ndarray:
    """-> ``(H, W, 3)`` uint8 RGB."""
    enc = (img.encoding or "jpeg").lower()
    if enc in ("jpeg", "jpg", "png"):
        from PIL import Image
        return np.asarray(Image.open(io.BytesIO(img.image_data)).convert("RGB"))
    if enc.startswith("raw"):
        # "raw" = square image; "raw:HxW" carries the geometry
        buf = np.frombuffer(img.image_data, dtype=np.uint8)
        if ":" in enc:
            h, w = (int(x) for x in enc.split(":", 1)[1].split("x"))
        else:
            side = int(round((buf.size // 3) ** 0.5))
            h = w = side
        if h * w * 3 != buf.size:
            raise ValueError(f"raw image of {buf.size} bytes does not match {h}x{w}x3")
        return buf.reshape(h, w, 3)
    raise ValueError(f"unknown image encoding {img.encoding!r}")


class RobotPolicyServicer(pb_grpc.RobotPolicyServiceServicer):
    def __init__(self, cfg: TrainPipelineConfig, policy=None, device: torch.device | None = None, planner=None):
        self.cfg = cfg
        self.device = device or torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.infer = InferenceThread()
        self.planner = planner
        self.policy = policy if policy is not None else self.infer.submit(self._load_policy).result()
        # before the warm-up requests, so that a checkpoint that cannot support the score fails at start-up
        from ...policies.accel import configure_accel
        from ...policies.candidates import configure_candidates
        self.accel_prefix = configure_accel(self.policy, cfg)
        # likewise: the critic is loaded, placed and smoke-called here, and the warm-up runs at the widened batch
        configure_candidates(self.policy, cfg)
        self.requests = 0
        self._lock = threading.Lock()
        for _ in range(cfg.server.warmup_requests if policy is None else 0):
            self.infer.submit(lambda: self._sample(self._dummy_batch(), None, 0)).result()

    # -- model ------------------------------------------------------------------------------------------
    def _load_policy(self):
        from ...policies.factory import make_policy
        policy = make_policy(self.cfg.policy).to(self.device)
        if self.device.type == "cuda":
            policy.to(torch.bfloat16)
            if self.cfg.server.use_cuda_graph and hasattr(policy, "enable_cuda_graphs"):
                policy.enable_cuda_graphs(True)
        return policy.eval()

    def _dummy_batch(self) -> dict[str, Any]:
        from ...configs.deployment import tag_norm_head
        from ...utils.utils import create_dummy_observation
        # warm-up takes the same head as real requests (a multi-head policy refuses an untagged batch)
        return tag_norm_head(create_dummy_observation(self.cfg, self.device), self.cfg.server)

    def _sample(self, batch, action_prefix, delay) -> torch.Tensor:
        with torch.inference_mode():
            return self.policy.sample_actions(batch, action_prefix=action_prefix, delay=delay)

    # -- request -> batch ---------------------------------------------------------------------------------
    def _prepare_observation(self, request) -> tuple[dict[str, Any], torch.Tensor | None, int]:
        cfg = self.cfg
        if not request.images:
            raise ValueError("the request carries no camera image")
        if len(request.images) > cfg.num_cams:
            raise ValueError(f"{len(request.images)} images sent, the policy takes {cfg.num_cams}")
        from ... import ops
        H, W = cfg.resolution
        batch: dict[str, Any] = {}
        pads = []
        for i in range(cfg.num_cams):
            if i < len(request.images):
                arr = decode_image(request.images[i])
                t = torch.from_numpy(np.ascontiguousarray(arr)).to(self.device).permute(2, 0, 1)[None].float() / 255.0
                if tuple(t.shape[-2:]) != (H, W):
                    t = ops.resize_with_pad(t, W, H, pad_value=0.0)
                batch[f"camera{i}"] = t
                pads.append(False)
            else:
                batch[f"camera{i}"] = torch.zeros(1, 3, H, W, device=self.device)
                pads.append(True)
        st = list(request.robot_state.state)
        if len(st) > cfg.max_state_dim:
            raise ValueError(f"state of {len(st)} values exceeds max_state_dim={cfg.max_state_dim}")
        state = torch.zeros(1, cfg.max_state_dim, device=self.device)
        state[0, :len(st)] = torch.tensor(st, device=self.device)
        batch["state"] = state
        batch["prompt"] = [request.prompt]
        batch["img_is_pad"] = torch.tensor([pads], dtype=torch.bool, device=self.device)
        prefix, delay = None, int(request.delay)
        if request.prefix_action:
            rows = [list(v.values) for v in request.prefix_action]
            if len(rows) > cfg.action_chunk:
                raise ValueError("prefix_action is longer than the action chunk")
            prefix = torch.zeros(1, cfg.action_chunk, cfg.max_action_dim, device=self.device)
            for j, r in enumerate(rows):
                prefix[0, j, :len(r)] = torch.tensor(r, device=self.device)
            if delay > len(rows):
                raise ValueError("delay exceeds the number of prefix actions")
        elif delay:
            raise ValueError("delay > 0 needs prefix_action")
        from ...configs.deployment import tag_norm_head
        tag_norm_head(batch, cfg.server)
        return batch, prefix, delay

    def _apply_planner(self, request, batch: dict[str, Any]) -> None:
        """The request prompt is the OVERALL task.  The planner sees every observation (its background loop replans
        from the latest one), the policy is prompted with the current subtask and never waits for the planner, except
        on the first request of a task, where one plan is computed in line so that the episode starts on a real
        subtask (a failing planner call leaves the overall task as the prompt)."""
        if self.planner is None:
            return
        task = request.prompt
        images = {k: v[0] for k, v in batch.items() if k.startswith("camera")}
        state = list(request.robot_state.state)
        sub = self.planner.current_subtask(task)          # resets the planner's memory when the task changed
        self.planner.observe(images, state)
        if not sub:
            try:
                sub = self.planner.plan(task, images, state).subtask
            except Exception as e:  # noqa: BLE001 - serving continues on the overall task
                logger.warning("first plan for %r failed: %s", task, e)
        if sub:
            batch["prompt"] = [sub]

    # -- RPCs ---------------------------------------------------------------------------------------------
    def _respond(self, request) -> "pb.ActionChunkResponse":
        t0 = time.perf_counter()
        resp = pb.ActionChunkResponse(request_id=request.request_id, timestamp_ns=time.time_ns())
        batch, prefix, delay = self._prepare_observation(request)
        self._apply_planner(request, batch)
        chunk = self.infer.submit(lambda: self._sample(batch, prefix, delay).squeeze(0).float().cpu()).result()
        accel = getattr(self.policy, "last_accel", None)
        if accel:
            resp.accel = float(accel[0])
        for row in chunk.numpy():
            resp.action_chunk.add(values=row.tolist())
        resp.inference_time_ms = (time.perf_counter() - t0) * 1e3
        with self._lock:
            self.requests += 1
        return resp

    def GetActionChunk(self, request, context):
        try:
            return self._respond(request)
        except ValueError as e:
            logger.error("Invalid request: %s", e)
            context.abort(grpc.StatusCode.INVALID_ARGUMENT, str(e))
        except Exception as e:  # noqa: BLE001
            logger.exception("Error during inference")
            context.abort(grpc.StatusCode.INTERNAL, f"Inference error: {type(e).__name__}: {e}")

    def StreamActionChunks(self, request_iterator: Iterator, context):
        for request in request_iterator:
            try:
                yield self._respond(request)
            except ValueError as e:
                context.abort(grpc.StatusCode.INVALID_ARGUMENT, str(e))
            except Exception as e:  # noqa: BLE001
                logger.exception("Error during streaming inference")
                context.abort(grpc.StatusCode.INTERNAL, f"Inference error: {type(e).__name__}: {e}")

    def HealthCheck(self, request, context):
        used = total = 0.0
        if self.device.type == "cuda":
            free, tot = torch.cuda.mem_get_info(self.device)
            used, total = (tot - free) / 1e9, tot / 1e9
        return pb.HealthCheckResponse(healthy=self.policy is not None, status="SERVING",
                                      model_name=getattr(self.cfg.policy, "type", "unknown"), device=str(self.device),
                                      gpu_memory_used_gb=used, gpu_memory_total_gb=total)


def build_server(cfg: TrainPipelineConfig, servicer: RobotPolicyServicer, port: int | None = None):
    s = cfg.server
    keys = load_api_keys([s.api_key] if s.api_key else None)
    import os
    if os.environ.get(s.api_key_env):
        keys.append(os.environ[s.api_key_env])
    interceptors = [ApiKeyInterceptor(keys)] if keys else []
    server = grpc.server(futures.ThreadPoolExecutor(max_workers=s.max_workers), interceptors=interceptors, options=[
        ("grpc.max_send_message_length", s.max_send_message_length_mb << 20),
        ("grpc.max_receive_message_length", s.max_receive_message_length_mb << 20)])
    pb_grpc.add_RobotPolicyServiceServicer_to_server(servicer, server)
    bound = server.add_insecure_port(f"127.0.0.1:{port if port is not None else s.port}" if port == 0
                                     else f"[::]:{port if port is not None else s.port}")
    return server, bound


@parser.wrap()
def serve(cfg: TrainPipelineConfig):
    from ...utils.logging_utils import init_logging
    init_logging()
    servicer = RobotPolicyServicer(cfg)
    server, port = build_server(cfg, servicer)
    server.start()
    logger.info("policy server listening on port %d (%s on %s)", port, cfg.policy.type, servicer.device)
    try:
        server.wait_for_termination()
    finally:
        servicer.infer.stop()


if __name__ == "__main__":
    serve()
