"""OpenTelemetry-style tracing with a no-dependency fallback (reference: vllm/tracing/__init__.py:66 ``init_tracer``,
:90 ``instrument``; tracing/otel.py:60-134). When the ``opentelemetry`` packages are absent, spans are recorded by an
in-process recorder with the same attribute names, so request spans (queue / prefill / decode times) stay testable."""
from __future__ import annotations

import contextlib
import functools
import time
from typing import Optional

_SPANS: list = []
_tracer = None
_enabled = False


class SpanAttributes:
    REQUEST_ID = "gen_ai.request.id"
    PROMPT_TOKENS = "gen_ai.usage.prompt_tokens"
    COMPLETION_TOKENS = "gen_ai.usage.completion_tokens"
    TIME_IN_QUEUE = "gen_ai.latency.time_in_queue"
    TTFT = "gen_ai.latency.time_to_first_token"
    E2E = "gen_ai.latency.e2e"


def init_tracer(name: str = "onecat_vllm", endpoint: Optional[str] = None):
    global _tracer, _enabled
    _enabled = True
    if endpoint:
        try:
            from opentelemetry import trace
            from opentelemetry.exporter.otlp.proto.grpc.trace_exporter import OTLPSpanExporter
            from opentelemetry.sdk.trace import TracerProvider
            from opentelemetry.sdk.trace.export import BatchSpanProcessor
            prov = TracerProvider()
            prov.add_span_processor(BatchSpanProcessor(OTLPSpanExporter(endpoint=endpoint)))
            trace.set_tracer_provider(prov)
            _tracer = trace.get_tracer(name)
        except ImportError:
            _tracer = None
    return _tracer


@contextlib.contextmanager
def span(name: str, **attrs):
    if not _enabled:
        yield None
        return
    if _tracer is not None:
        with _tracer.start_as_current_span(name) as sp:
            for k, v in attrs.items():
                sp.set_attribute(k, v)
            yield sp
        return
    rec = {"name": name, "start": time.time(), "attrs": dict(attrs)}
    try:
        yield rec
    finally:
        rec["end"] = time.time()
        _SPANS.append(rec)


def instrument(span_name: Optional[str] = None):
    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*a, **k):
            with span(span_name or fn.__qualname__):
                return fn(*a, **k)
        return wrapper
    return deco


def record_request_span(request_id: str, metrics, n_prompt: int, n_out: int) -> None:
    if not _enabled:
        return
    a = SpanAttributes
    attrs = {a.REQUEST_ID: request_id, a.PROMPT_TOKENS: n_prompt, a.COMPLETION_TOKENS: n_out}
    if metrics.first_token_time is not None:
        attrs[a.TTFT] = metrics.first_token_time - metrics.arrival_time
    if metrics.finished_time is not None:
        attrs[a.E2E] = metrics.finished_time - metrics.arrival_time
    with span("llm_request", **attrs):
        pass


def recorded_spans() -> list:
    return list(_SPANS)


def extract_trace_headers(headers: dict) -> dict:
    return {k: v for k, v in headers.items() if k.lower() in ("traceparent", "tracestate")}
