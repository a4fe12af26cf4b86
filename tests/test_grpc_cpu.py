"""gRPC policy server on the loopback interface with a tiny pi0.5: chunk shape, request validation, streaming,
health check, API-key enforcement, and wire compatibility of the hand-built message classes."""

import numpy as np
import pytest

grpc = pytest.importorskip("grpc")

from helpers import TINY  # noqa: E402
from opentau_b200.configs.train import TrainPipelineConfig  # noqa: E402
from opentau_b200.scripts.grpc import robot_inference_pb2 as pb  # noqa: E402
from opentau_b200.scripts.grpc.client import PolicyClient  # noqa: E402
from opentau_b200.scripts.grpc.server import RobotPolicyServicer, build_server  # noqa: E402


def _cfg(path, **server):
    return TrainPipelineConfig.from_dict({
        "policy": {"type": "pi05", "pretrained_path": str(path), "chunk_size": 10, "n_action_steps": 10, "prompt_max_length": 24, "dropout": 0.0,
                   "discrete_action_max_length": 8, "discrete_action_vocab_size": 256, "device": "cpu", "num_steps": 2,
                   "max_delay": 3,
                   "input_features": {"camera0": {"type": "VISUAL", "shape": [3, 224, 224]},
                                      "state": {"type": "STATE", "shape": [32]}},
                   "output_features": {"actions": {"type": "ACTION", "shape": [32]}}, **TINY},
        "resolution": [224, 224], "num_cams": 1, "action_chunk": 10, "batch_size": 1,
        "server": {"port": 50999, "warmup_requests": 1, **server}})


@pytest.fixture()
def running(tmp_path):
    from helpers import tiny_pi05
    tiny_pi05(num_steps=2, max_delay=3, prompt_max_length=24).save_pretrained(tmp_path / "ckpt")

    def start(**server):
        cfg = _cfg(tmp_path / "ckpt", **server)
        svc = RobotPolicyServicer(cfg)
        srv, port = build_server(cfg, svc, port=0)
        srv.start()
        started.append((srv, svc))
        return port
    started = []
    yield start
    for srv, svc in started:
        srv.stop(0)
        svc.infer.stop()


def test_action_chunk_stream_and_health(running):
    port = running()
    c = PolicyClient(f"127.0.0.1:{port}")
    h = c.health()
    assert h.healthy and h.model_name == "pi05" and h.device == "cpu"
    img = np.random.default_rng(0).integers(0, 255, (120, 160, 3), dtype=np.uint8)
    chunk, resp = c.get_action_chunk([img], np.zeros(7), "pick up the block")
    assert chunk.shape == (10, 32) and np.isfinite(chunk).all() and resp.inference_time_ms > 0 and resp.request_id
    assert not resp.HasField("accel")
    # real-time chunking: 3 leftover actions, 2 of them frozen
    chunk2, _ = c.get_action_chunk([img], np.zeros(7), "pick up the block", prefix_action=chunk[:3], delay=2,
                                   encoding="raw")
    assert chunk2.shape == (10, 32)
    outs = list(c.stream([c.make_request([img], np.zeros(7), "a"), c.make_request([img], np.zeros(7), "b", encoding="png")]))
    assert len(outs) == 2 and outs[1][0].shape == (10, 32)
    with pytest.raises(grpc.RpcError) as e:
        c.get_action_chunk([], np.zeros(7), "no image")
    assert e.value.code() == grpc.StatusCode.INVALID_ARGUMENT
    with pytest.raises(grpc.RpcError) as e:
        c.get_action_chunk([img], np.zeros(40), "state too wide")
    assert e.value.code() == grpc.StatusCode.INVALID_ARGUMENT
    c.close()


def test_api_key_is_enforced(running):
    port = running(api_key="s3cret")
    img = np.zeros((64, 64, 3), np.uint8)
    anon = PolicyClient(f"127.0.0.1:{port}")
    assert anon.health().healthy                               # health stays open
    with pytest.raises(grpc.RpcError) as e:
        anon.get_action_chunk([img], np.zeros(4), "x")
    assert e.value.code() == grpc.StatusCode.UNAUTHENTICATED
    chunk, _ = PolicyClient(f"127.0.0.1:{port}", api_key="s3cret").get_action_chunk([img], np.zeros(4), "x")
    assert chunk.shape == (10, 32)


def test_wire_format_matches_the_proto_field_numbers():
    r = pb.ObservationRequest(prompt="hi", delay=2, request_id="r")
    r.robot_state.state.extend([1.0, 2.0])
    raw = r.SerializeToString()
    # field 3 (prompt) = tag 0x1a, field 5 (delay) = tag 0x28, field 7 (request_id) = tag 0x3a
    assert b"\x1a\x02hi" in raw and b"\x28\x02" in raw and b"\x3a\x01r" in raw
    assert pb.ObservationRequest.FromString(raw).robot_state.state == [1.0, 2.0]


def test_planner_sees_observations_and_sets_the_subtask(tmp_path):
    """With a planner attached the request prompt is the overall task: the first request plans in line, every request
    feeds the planner's observation cache, and the policy is prompted with the planner's subtask."""
    from helpers import tiny_pi05
    from opentau_b200.planner.high_level_planner import CallableClient, SubtaskPlanner
    tiny_pi05(num_steps=2, max_delay=3, prompt_max_length=24).save_pretrained(tmp_path / "ckpt")
    calls = []

    def model(messages, images):
        calls.append((messages[-1]["content"], len(images)))
        return "Updated Memory: started\nSubtask: open the drawer"

    planner = SubtaskPlanner(CallableClient(model))
    svc = RobotPolicyServicer(_cfg(tmp_path / "ckpt"), planner=planner)
    seen = []
    real_sample = svc._sample
    svc._sample = lambda batch, prefix, delay: (seen.append(batch["prompt"][0]), real_sample(batch, prefix, delay))[1]
    try:
        img = np.zeros((32, 32, 3), np.uint8)
        req = PolicyClient.make_request(None, [img], np.arange(3, dtype=np.float32), "tidy the desk")
        resp = svc._respond(req)
        assert len(resp.action_chunk) == 10 and seen[-1] == "open the drawer"
        assert len(calls) == 1 and calls[0][1] == 1 and "tidy the desk" in calls[0][0]
        assert planner._latest is not None and list(planner._latest[1]) == [0.0, 1.0, 2.0]
        svc._respond(req)                                   # the subtask is cached: no further in-line call
        assert len(calls) == 1 and seen[-1] == "open the drawer"
        svc._respond(PolicyClient.make_request(None, [img], np.zeros(3, np.float32), "water the plant"))
        assert len(calls) == 2 and "water the plant" in calls[1][0]        # a new task plans afresh
    finally:
        svc.infer.stop()


def test_robot_control_loop_and_client_retries(running):
    from opentau_b200.scripts.grpc.client import ClientConfig, RobotControlLoop, RobotLoopConfig
    port = running()
    sent = []
    joints = tuple(f"j{i}" for i in range(4))
    cfg = RobotLoopConfig(server_address=f"127.0.0.1:{port}", num_cameras=1, joint_names=joints)
    loop = RobotControlLoop(cfg, publish=lambda names, q: sent.append((names, q)))
    assert loop.step() == "no_state" and not sent
    assert loop.on_joint_state([0.1, 0.2], [0.0, 0.0]) is False and loop.last_status == "short_state"
    assert loop.on_joint_state([0.1, 0.2, 0.3, 0.4, 9.0], [0.0] * 5) and loop.positions == [0.1, 0.2, 0.3, 0.4]
    assert loop.step() == "no_prompt" and not sent
    cfg.prompt = "pick up the block"
    assert loop.step() == "ok" and len(sent) == 1 and sent[0][0] == joints and len(sent[0][1]) == 4
    assert loop.last_inference_ms > 0
    # the command is the LAST row of the chunk; malformed chunks publish nothing
    assert loop.apply(np.arange(12, dtype=np.float32).reshape(3, 4)) == "ok" and sent[-1][1] == [8.0, 9.0, 10.0, 11.0]
    assert loop.apply(np.zeros((0, 4), np.float32)) == "empty_chunk"
    assert loop.apply(np.zeros((2, 3), np.float32)) == "short_action"
    assert loop.apply(np.zeros((1, 2, 3), np.float32)) == "bad_chunk" and len(sent) == 2
    health = loop.client.health_check()
    assert health["healthy"] and health["model_name"] == "pi05"
    loop.stop()                                                       # damping: hold the current positions
    assert sent[-1][1] == [0.1, 0.2, 0.3, 0.4] and not loop.client.is_connected()
    assert loop.step() == "not_connected" and loop.client.health_check() == {"healthy": False, "status": "not connected"}
    # a dead address: bounded retries, then one error
    from opentau_b200.scripts.grpc.client import PolicyClient as C
    dead = C(ClientConfig(server_address="127.0.0.1:1", timeout_seconds=0.3, max_retries=2, retry_delay_seconds=0.01))
    with pytest.raises(RuntimeError, match="after 2 attempts"):
        dead.request_action_chunk([np.zeros((8, 8, 3), np.uint8)], np.zeros(3), "x")
    assert dead.health_check()["healthy"] is False
    assert dead.connect(wait_ready_s=0.2) is False
    with pytest.raises(ValueError):
        ClientConfig(max_retries=0)
