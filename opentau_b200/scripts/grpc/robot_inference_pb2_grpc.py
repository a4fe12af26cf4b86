"""Client stub and server registration for ``robot_inference.RobotPolicyService`` (same shape as protoc output)."""

from __future__ import annotations

import grpc

from . import robot_inference_pb2 as pb

_SVC = "robot_inference.RobotPolicyService"


class RobotPolicyServiceStub:
    def __init__(self, channel: grpc.Channel):
        self.GetActionChunk = channel.unary_unary(
            f"/{_SVC}/GetActionChunk", request_serializer=pb.ObservationRequest.SerializeToString,
            response_deserializer=pb.ActionChunkResponse.FromString)
        self.StreamActionChunks = channel.stream_stream(
            f"/{_SVC}/StreamActionChunks", request_serializer=pb.ObservationRequest.SerializeToString,
            response_deserializer=pb.ActionChunkResponse.FromString)
        self.HealthCheck = channel.unary_unary(
            f"/{_SVC}/HealthCheck", request_serializer=pb.HealthCheckRequest.SerializeToString,
            response_deserializer=pb.HealthCheckResponse.FromString)


class RobotPolicyServiceServicer:
    def GetActionChunk(self, request, context):
        context.set_code(grpc.StatusCode.UNIMPLEMENTED)
        raise NotImplementedError("Method not implemented!")

    def StreamActionChunks(self, request_iterator, context):
        context.set_code(grpc.StatusCode.UNIMPLEMENTED)
        raise NotImplementedError("Method not implemented!")

    def HealthCheck(self, request, context):
        context.set_code(grpc.StatusCode.UNIMPLEMENTED)
        raise NotImplementedError("Method not implemented!")


def add_RobotPolicyServiceServicer_to_server(servicer, server) -> None:
    handlers = {
        "GetActionChunk": grpc.unary_unary_rpc_method_handler(
            servicer.GetActionChunk, request_deserializer=pb.ObservationRequest.FromString,
            response_serializer=pb.ActionChunkResponse.SerializeToString),
        "StreamActionChunks": grpc.stream_stream_rpc_method_handler(
            servicer.StreamActionChunks, request_deserializer=pb.ObservationRequest.FromString,
            response_serializer=pb.ActionChunkResponse.SerializeToString),
        "HealthCheck": grpc.unary_unary_rpc_method_handler(
            servicer.HealthCheck, request_deserializer=pb.HealthCheckRequest.FromString,
            response_serializer=pb.HealthCheckResponse.SerializeToString),
    }
    server.add_generic_rpc_handlers((grpc.method_handlers_generic_handler(_SVC, handlers),))
