"""Request tracing (counterpart of vllm/tracing.py:51-120): one span per finished request with the
queue time, time to first token, end-to-end latency and token counts as attributes. Spans go to an
OpenTelemetry OTLP exporter when the ``opentelemetry`` packages are installed and an endpoint is given,
otherwise to a JSON-lines file (or nowhere). ``trace_function_calls`` is the ``TW_TRACE_FUNCTION``
debugging aid: it logs every Python call and return inside the package (vllm/logger.py:151-210)."""
from __future__ import annotations

import json
import os
import sys
import threading
import time
from typing import Optional

from ..outputs import RequestOutput

SPAN_ATTRS = ("gen_ai.request.id", "gen_ai.usage.prompt_tokens", "gen_ai.usage.completion_tokens",
              "gen_ai.latency.time_in_queue", "gen_ai.latency.time_to_first_token", "gen_ai.latency.e2e")


class RequestTracer:
    def __init__(self, otlp_endpoint: Optional[str] = None, jsonl_path: Optional[str] = None,
                 service_name: str = "tokenweave_b200"):
        self._otel = None
        self._file = None
        self._lock = threading.Lock()
        if otlp_endpoint:
            try:
                from opentelemetry import trace
                from opentelemetry.exporter.otlp.proto.grpc.trace_exporter import OTLPSpanExporter
                from opentelemetry.sdk.resources import Resource
                from opentelemetry.sdk.trace import TracerProvider
                from opentelemetry.sdk.trace.export import BatchSpanProcessor
                provider = TracerProvider(resource=Resource.create({"service.name": service_name}))
                provider.add_span_processor(BatchSpanProcessor(OTLPSpanExporter(endpoint=otlp_endpoint)))
                trace.set_tracer_provider(provider)
                self._otel = trace.get_tracer(service_name)
            except ImportError:
                jsonl_path = jsonl_path or "tokenweave_traces.jsonl"
        if self._otel is None and jsonl_path:
            self._file = open(jsonl_path, "a")

    @staticmethod
    def attributes(out: RequestOutput) -> dict:
        m = out.metrics
        n_out = sum(len(c.token_ids) for c in out.outputs)
        return {
            "gen_ai.request.id": out.request_id,
            "gen_ai.usage.prompt_tokens": len(out.prompt_token_ids),
            "gen_ai.usage.completion_tokens": n_out,
            "gen_ai.latency.time_in_queue": (m.first_scheduled_time - m.arrival_time) if m.first_scheduled_time else None,
            "gen_ai.latency.time_to_first_token": (m.first_token_time - m.arrival_time) if m.first_token_time else None,
            "gen_ai.latency.e2e": (m.finished_time - m.arrival_time) if m.finished_time else None,
        }

    def record(self, out: RequestOutput) -> None:
        if not out.finished:
            return
        attrs = self.attributes(out)
        if self._otel is not None:
            with self._otel.start_as_current_span("llm_request") as span:
                for k, v in attrs.items():
                    if v is not None:
                        span.set_attribute(k, v)
        elif self._file is not None:
            with self._lock:
                self._file.write(json.dumps({"name": "llm_request", "time": time.time(), "attributes": attrs}) + "\n")
                self._file.flush()

    def close(self) -> None:
        if self._file is not None:
            self._file.close()
            self._file = None


def trace_function_calls(log_path: str, root_dir: Optional[str] = None) -> None:
    """Log every call and return of Python functions defined under ``root_dir`` (default: this package)."""
    root_dir = root_dir or os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    f = open(log_path, "a")

    def tracer(frame, event, arg):
        if event in ("call", "return"):
            code = frame.f_code
            if code.co_filename.startswith(root_dir):
                f.write(f"{time.time():.6f} {event} {code.co_name} {code.co_filename}:{frame.f_lineno}\n")
                f.flush()
        return tracer

    sys.settrace(tracer)
    threading.settrace(tracer)
