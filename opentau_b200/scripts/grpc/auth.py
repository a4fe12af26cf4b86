"""API-key authentication for the policy server (reference ``src/opentau/scripts/grpc/auth.py:30-112``): a server
interceptor that rejects calls whose ``x-api-key`` (or ``authorization: Bearer``) metadata does not match; the
health check may stay open."""

from __future__ import annotations

import hmac
import os

import grpc

API_KEY_HEADER = "x-api-key"
API_KEY_ENV = "OPENTAU_GRPC_API_KEY"


def load_api_keys(keys: list[str] | None = None) -> list[str]:
    out = [k for k in (keys or []) if k]
    env = os.environ.get(API_KEY_ENV, "")
    out += [k.strip() for k in env.split(",") if k.strip()]
    return out


class ApiKeyInterceptor(grpc.ServerInterceptor):
    def __init__(self, keys: list[str], open_methods: tuple[str, ...] = ("HealthCheck",)):
        if not keys:
            raise ValueError("ApiKeyInterceptor needs at least one key")
        self.keys = [k.encode() for k in keys]
        self.open_methods = open_methods

        def deny(request, context):
            context.abort(grpc.StatusCode.UNAUTHENTICATED, "invalid or missing API key")

        def deny_stream(request_iterator, context):
            context.abort(grpc.StatusCode.UNAUTHENTICATED, "invalid or missing API key")

        self._deny_unary = grpc.unary_unary_rpc_method_handler(deny)
        self._deny_stream = grpc.stream_stream_rpc_method_handler(deny_stream)

    def _ok(self, metadata) -> bool:
        md = {k.lower(): v for k, v in metadata}
        cand = md.get(API_KEY_HEADER)
        if cand is None and md.get("authorization", "").lower().startswith("bearer "):
            cand = md["authorization"][7:]
        if cand is None:
            return False
        c = cand.encode() if isinstance(cand, str) else cand
        return any(hmac.compare_digest(c, k) for k in self.keys)

    def intercept_service(self, continuation, handler_call_details):
        method = handler_call_details.method.rsplit("/", 1)[-1]
        if method in self.open_methods or self._ok(handler_call_details.invocation_metadata):
            return continuation(handler_call_details)
        return self._deny_stream if method == "StreamActionChunks" else self._deny_unary


class ApiKeyClientInterceptor(grpc.UnaryUnaryClientInterceptor, grpc.StreamStreamClientInterceptor):
    """Adds the key to every outgoing call."""

    def __init__(self, key: str):
        self.key = key

    def _details(self, d):
        md = list(d.metadata or []) + [(API_KEY_HEADER, self.key)]
        return d._replace(metadata=md) if hasattr(d, "_replace") else _Details(d, md)

    def intercept_unary_unary(self, continuation, client_call_details, request):
        return continuation(self._details(client_call_details), request)

    def intercept_stream_stream(self, continuation, client_call_details, request_iterator):
        return continuation(self._details(client_call_details), request_iterator)


class _Details(grpc.ClientCallDetails):
    def __init__(self, d, metadata):
        self.method, self.timeout, self.metadata = d.method, d.timeout, metadata
        self.credentials = d.credentials
        self.wait_for_ready = getattr(d, "wait_for_ready", None)
        self.compression = getattr(d, "compression", None)
