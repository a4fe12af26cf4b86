"""Message classes of ``robot_inference.proto``, built at import time from a descriptor written out in Python
(no protoc run needed; wire compatible with stubs generated from the .proto file)."""

from __future__ import annotations

from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

_F = descriptor_pb2.FieldDescriptorProto
_PKG = "robot_inference"


def _field(name, number, ftype, label=_F.LABEL_OPTIONAL, type_name=None, proto3_optional=False, oneof_index=None):
    f = _F(name=name, number=number, type=ftype, label=label)
    if type_name:
        f.type_name = f".{_PKG}.{type_name}"
    if proto3_optional:
        f.proto3_optional = True
        f.oneof_index = oneof_index
    return f


def _build() -> descriptor_pb2.FileDescriptorProto:
    fd = descriptor_pb2.FileDescriptorProto(name="robot_inference.proto", package=_PKG, syntax="proto3")
    R = _F.LABEL_REPEATED
    m = fd.message_type.add(name="CameraImage")
    m.field.extend([_field("image_data", 1, _F.TYPE_BYTES), _field("encoding", 2, _F.TYPE_STRING)])
    m = fd.message_type.add(name="RobotState")
    m.field.extend([_field("state", 1, _F.TYPE_FLOAT, R)])
    m = fd.message_type.add(name="ActionVector")
    m.field.extend([_field("values", 1, _F.TYPE_FLOAT, R)])
    m = fd.message_type.add(name="ObservationRequest")
    m.field.extend([_field("images", 1, _F.TYPE_MESSAGE, R, "CameraImage"),
                    _field("robot_state", 2, _F.TYPE_MESSAGE, type_name="RobotState"),
                    _field("prompt", 3, _F.TYPE_STRING), _field("prefix_action", 4, _F.TYPE_MESSAGE, R, "ActionVector"),
                    _field("delay", 5, _F.TYPE_INT32), _field("timestamp_ns", 6, _F.TYPE_INT64),
                    _field("request_id", 7, _F.TYPE_STRING)])
    m = fd.message_type.add(name="ActionChunkResponse")
    m.oneof_decl.add(name="_accel")
    m.field.extend([_field("action_chunk", 1, _F.TYPE_MESSAGE, R, "ActionVector"),
                    _field("timestamp_ns", 2, _F.TYPE_INT64), _field("request_id", 3, _F.TYPE_STRING),
                    _field("inference_time_ms", 4, _F.TYPE_FLOAT),
                    _field("accel", 5, _F.TYPE_FLOAT, proto3_optional=True, oneof_index=0)])
    fd.message_type.add(name="HealthCheckRequest")
    m = fd.message_type.add(name="HealthCheckResponse")
    m.field.extend([_field("healthy", 1, _F.TYPE_BOOL), _field("status", 2, _F.TYPE_STRING),
                    _field("model_name", 3, _F.TYPE_STRING), _field("device", 4, _F.TYPE_STRING),
                    _field("gpu_memory_used_gb", 5, _F.TYPE_FLOAT), _field("gpu_memory_total_gb", 6, _F.TYPE_FLOAT)])
    svc = fd.service.add(name="RobotPolicyService")
    svc.method.add(name="GetActionChunk", input_type=f".{_PKG}.ObservationRequest",
                   output_type=f".{_PKG}.ActionChunkResponse")
    svc.method.add(name="StreamActionChunks", input_type=f".{_PKG}.ObservationRequest",
                   output_type=f".{_PKG}.ActionChunkResponse", client_streaming=True, server_streaming=True)
    svc.method.add(name="HealthCheck", input_type=f".{_PKG}.HealthCheckRequest",
                   output_type=f".{_PKG}.HealthCheckResponse")
    return fd


_pool = descriptor_pool.DescriptorPool()
DESCRIPTOR = _pool.Add(_build())


def _cls(name: str):
    return message_factory.GetMessageClass(_pool.FindMessageTypeByName(f"{_PKG}.{name}"))


CameraImage = _cls("CameraImage")
RobotState = _cls("RobotState")
ActionVector = _cls("ActionVector")
ObservationRequest = _cls("ObservationRequest")
ActionChunkResponse = _cls("ActionChunkResponse")
HealthCheckRequest = _cls("HealthCheckRequest")
HealthCheckResponse = _cls("HealthCheckResponse")
