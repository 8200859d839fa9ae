"""Stat loggers: periodic log line, Prometheus series, in-memory snapshot
(reference: vllm/v1/metrics/loggers.py:99 ``LoggingStatLogger``, :404 ``PrometheusStatLogger`` with series names :452-1024;
v1/metrics/stats.py:171,325; v1/metrics/reader.py for ``LLM.get_metrics``)."""
from __future__ import annotations

import time
from typing import Optional

from onecat_vllm.logger import init_logger

log = init_logger(__name__)

_TTFT_BUCKETS = [0.001, 0.005, 0.01, 0.02, 0.04, 0.06, 0.08, 0.1, 0.25, 0.5, 0.75, 1.0, 2.5, 5.0, 7.5, 10.0, 20.0, 40.0, 80.0, 160.0, 640.0, 2560.0]
_ITL_BUCKETS = [0.01, 0.025, 0.05, 0.075, 0.1, 0.15, 0.2, 0.3, 0.4, 0.5, 0.75, 1.0, 2.5, 5.0, 7.5, 10.0, 20.0, 40.0, 80.0]


class StatLoggerBase:
    def record(self, scheduler_stats, outputs: list, finished: list) -> None:
        raise NotImplementedError

    def snapshot(self) -> dict:
        return {}


class AggregateStatLogger(StatLoggerBase):
    """Keeps running totals; the base for the log line and for ``get_metrics``."""

    def __init__(self):
        self.t0 = time.monotonic()
        self.num_generation_tokens = 0
        self.num_prompt_tokens = 0
        self.num_preemptions = 0
        self.prefix_queries = self.prefix_hits = 0
        self.num_finished = 0
        self.spec_drafts = self.spec_draft_tokens = self.spec_accepted = 0
        self.last = None
        self.ttft: list = []
        self.tpot: list = []
        self.e2e: list = []
        self.step_device_ms = 0.0
        self.steps = 0

    def record(self, s, outputs, finished):
        self.last = s
        self.steps += 1
        self.num_generation_tokens += sum(len(o.new_token_ids) for o in outputs)
        self.num_preemptions += s.num_preemptions
        self.prefix_queries += s.prefix_cache_queries
        self.prefix_hits += s.prefix_cache_hits
        self.spec_drafts += s.spec_num_drafts
        self.spec_draft_tokens += s.spec_num_draft_tokens
        self.spec_accepted += s.spec_num_accepted_tokens
        self.step_device_ms += s.step_device_ms
        for m in finished:
            self.num_finished += 1
            if m.first_token_time is not None:
                self.ttft.append(m.first_token_time - m.arrival_time)
            if m.finished_time is not None:
                self.e2e.append(m.finished_time - m.arrival_time)

    def snapshot(self) -> dict:
        s = self.last
        el = max(time.monotonic() - self.t0, 1e-9)
        return {
            "vllm:num_requests_running": s.num_running_reqs if s else 0,
            "vllm:num_requests_waiting": s.num_waiting_reqs if s else 0,
            "vllm:kv_cache_usage_perc": s.kv_cache_usage if s else 0.0,
            "vllm:generation_tokens_total": self.num_generation_tokens,
            "vllm:num_preemptions_total": self.num_preemptions,
            "vllm:prefix_cache_queries_total": self.prefix_queries,
            "vllm:prefix_cache_hits_total": self.prefix_hits,
            "vllm:request_success_total": self.num_finished,
            "vllm:spec_decode_num_drafts_total": self.spec_drafts,
            "vllm:spec_decode_num_draft_tokens_total": self.spec_draft_tokens,
            "vllm:spec_decode_num_accepted_tokens_total": self.spec_accepted,
            "vllm:avg_generation_throughput_toks_per_s": self.num_generation_tokens / el,
            "vllm:time_to_first_token_seconds_p50": sorted(self.ttft)[len(self.ttft) // 2] if self.ttft else None,
            "vllm:e2e_request_latency_seconds_p50": sorted(self.e2e)[len(self.e2e) // 2] if self.e2e else None,
            "onecat:step_device_ms_mean": self.step_device_ms / max(self.steps, 1),
        }


class LoggingStatLogger(AggregateStatLogger):
    def __init__(self, interval_s: float = 10.0):
        super().__init__()
        self.interval, self._last_log, self._tok_at_log = interval_s, time.monotonic(), 0

    def record(self, s, outputs, finished):
        super().record(s, outputs, finished)
        now = time.monotonic()
        if now - self._last_log >= self.interval:
            dt = now - self._last_log
            tput = (self.num_generation_tokens - self._tok_at_log) / dt
            hit = self.prefix_hits / self.prefix_queries if self.prefix_queries else 0.0
            log.info(f"gen throughput {tput:.1f} tok/s, running {s.num_running_reqs}, waiting {s.num_waiting_reqs}, "
                     f"KV usage {s.kv_cache_usage * 100:.1f}%, prefix hit rate {hit * 100:.1f}%")
            self._last_log, self._tok_at_log = now, self.num_generation_tokens


class PrometheusStatLogger(StatLoggerBase):
    """Exports the reference's ``vllm:*`` series names so existing dashboards keep working."""

    _singleton = None

    def __init__(self, model_name: str = "model"):
        import prometheus_client as pc
        lab = ["model_name"]
        self.lv = [model_name]
        mk = lambda cls, name, doc, **kw: cls(name, doc, lab, **kw)
        self.g_running = mk(pc.Gauge, "vllm:num_requests_running", "requests in the running queue")
        self.g_waiting = mk(pc.Gauge, "vllm:num_requests_waiting", "requests waiting to be scheduled")
        self.g_kv = mk(pc.Gauge, "vllm:kv_cache_usage_perc", "fraction of KV blocks in use")
        self.c_gen = mk(pc.Counter, "vllm:generation_tokens", "generated tokens")
        self.c_prompt = mk(pc.Counter, "vllm:prompt_tokens", "prefilled tokens")
        self.c_preempt = mk(pc.Counter, "vllm:num_preemptions", "preemptions")
        self.c_pq = mk(pc.Counter, "vllm:prefix_cache_queries", "prefix cache queried tokens")
        self.c_ph = mk(pc.Counter, "vllm:prefix_cache_hits", "prefix cache hit tokens")
        self.c_ok = mk(pc.Counter, "vllm:request_success", "finished requests")
        self.c_drafts = mk(pc.Counter, "vllm:spec_decode_num_drafts", "speculative drafts")
        self.c_dtok = mk(pc.Counter, "vllm:spec_decode_num_draft_tokens", "draft tokens")
        self.c_acc = mk(pc.Counter, "vllm:spec_decode_num_accepted_tokens", "accepted draft tokens")
        self.h_ttft = mk(pc.Histogram, "vllm:time_to_first_token_seconds", "TTFT", buckets=_TTFT_BUCKETS)
        self.h_itl = mk(pc.Histogram, "vllm:inter_token_latency_seconds", "inter-token latency", buckets=_ITL_BUCKETS)
        self.h_tpot = mk(pc.Histogram, "vllm:request_time_per_output_token_seconds", "TPOT", buckets=_ITL_BUCKETS)
        self.h_e2e = mk(pc.Histogram, "vllm:e2e_request_latency_seconds", "request latency", buckets=_TTFT_BUCKETS)
        self.h_step = mk(pc.Histogram, "onecat:step_device_seconds", "device time of one engine step", buckets=_ITL_BUCKETS)
        tok_buckets = [1, 2, 5, 10, 20, 50, 100, 200, 500, 1000, 2000, 5000, 10000, 20000, 50000, 100000, 200000]
        self.h_iter_tokens = mk(pc.Histogram, "vllm:iteration_tokens_total", "tokens scheduled per engine step", buckets=tok_buckets)
        self.h_req_prompt = mk(pc.Histogram, "vllm:request_prompt_tokens", "prompt tokens per request", buckets=tok_buckets)
        self.h_req_gen = mk(pc.Histogram, "vllm:request_generation_tokens", "generated tokens per request", buckets=tok_buckets)
        self.h_req_max = mk(pc.Histogram, "vllm:request_params_max_tokens", "max_tokens per request", buckets=tok_buckets)
        self.h_queue = mk(pc.Histogram, "vllm:request_queue_time_seconds", "arrival to first schedule", buckets=_TTFT_BUCKETS)
        self.h_prefill = mk(pc.Histogram, "vllm:request_prefill_time_seconds", "first schedule to first token", buckets=_TTFT_BUCKETS)
        self.h_decode = mk(pc.Histogram, "vllm:request_decode_time_seconds", "first token to last token", buckets=_TTFT_BUCKETS)
        self.h_infer = mk(pc.Histogram, "vllm:request_inference_time_seconds", "first schedule to last token", buckets=_TTFT_BUCKETS)
        self.c_cached = mk(pc.Counter, "vllm:prompt_tokens_cached", "prompt tokens served from the prefix cache")
        self.c_reason = pc.Counter("vllm:request_finished", "finished requests by reason", lab + ["finished_reason"])
        self._last_tok_time: Optional[float] = None

    @classmethod
    def get(cls, model_name: str = "model") -> "PrometheusStatLogger":
        if cls._singleton is None:
            cls._singleton = cls(model_name)
        return cls._singleton

    def record(self, s, outputs, finished):
        lv = self.lv
        self.g_running.labels(*lv).set(s.num_running_reqs)
        self.g_waiting.labels(*lv).set(s.num_waiting_reqs)
        self.g_kv.labels(*lv).set(s.kv_cache_usage)
        n = sum(len(o.new_token_ids) for o in outputs)
        self.c_gen.labels(*lv).inc(n)
        self.c_preempt.labels(*lv).inc(s.num_preemptions)
        self.c_pq.labels(*lv).inc(s.prefix_cache_queries)
        self.c_ph.labels(*lv).inc(s.prefix_cache_hits)
        self.c_drafts.labels(*lv).inc(s.spec_num_drafts)
        self.c_dtok.labels(*lv).inc(s.spec_num_draft_tokens)
        self.c_acc.labels(*lv).inc(s.spec_num_accepted_tokens)
        if s.step_device_ms:
            self.h_step.labels(*lv).observe(s.step_device_ms / 1e3)
        now = time.monotonic()
        if n and self._last_tok_time is not None:
            self.h_itl.labels(*lv).observe(now - self._last_tok_time)
        if n:
            self._last_tok_time = now
        if s.num_scheduled_tokens:
            self.h_iter_tokens.labels(*lv).observe(s.num_scheduled_tokens)
        for m in finished:
            self.c_ok.labels(*lv).inc()
            self.c_reason.labels(*lv, m.finish_reason or "unknown").inc()
            self.c_prompt.labels(*lv).inc(m.num_prompt_tokens)
            self.c_cached.labels(*lv).inc(max(m.num_cached_tokens, 0))
            self.h_req_prompt.labels(*lv).observe(m.num_prompt_tokens)
            self.h_req_gen.labels(*lv).observe(m.num_generation_tokens)
            if m.max_tokens:
                self.h_req_max.labels(*lv).observe(m.max_tokens)
            first_sched = m.first_scheduled_time if m.first_scheduled_time is not None else m.arrival_time
            self.h_queue.labels(*lv).observe(max(first_sched - m.arrival_time, 0.0))
            if m.first_token_time is not None:
                self.h_ttft.labels(*lv).observe(max(m.first_token_time - m.arrival_time, 0.0))
                self.h_prefill.labels(*lv).observe(max(m.first_token_time - first_sched, 0.0))
            if m.finished_time is not None:
                self.h_e2e.labels(*lv).observe(max(m.finished_time - m.arrival_time, 0.0))
                self.h_infer.labels(*lv).observe(max(m.finished_time - first_sched, 0.0))
                if m.first_token_time is not None:
                    dec = max(m.finished_time - m.first_token_time, 0.0)
                    self.h_decode.labels(*lv).observe(dec)
                    if m.num_generation_tokens > 1:
                        self.h_tpot.labels(*lv).observe(dec / (m.num_generation_tokens - 1))


def make_stat_loggers(cfg, prometheus: bool = False) -> list:
    out: list = [LoggingStatLogger(cfg.observability_config.log_stats_interval_s)]
    if prometheus:
        out.append(PrometheusStatLogger.get(cfg.model_config.model))
    return out


def snapshot(loggers: list) -> dict:
    d: dict = {}
    for l in loggers:
        d.update(l.snapshot())
    return d
