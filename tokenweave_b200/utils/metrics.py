"""Step statistics and loggers (counterpart of vllm/v1/metrics/stats.py and loggers.py:33-445)."""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Optional

from .logging import init_logger

logger = init_logger(__name__)


@dataclass
class StepStats:
    num_tokens: int = 0
    num_running: int = 0
    num_waiting: int = 0
    kv_usage: float = 0.0
    num_generated: int = 0
    # cumulative counters of the engine (prefix cache in blocks, speculative decoding in tokens)
    prefix_cache_queries: int = 0
    prefix_cache_hits: int = 0
    num_draft_tokens: int = 0
    num_accepted_tokens: int = 0


class LoggingStatLogger:
    """Periodic throughput / queue / KV-usage line, like the reference's LoggingStatLogger."""

    def __init__(self, interval_s: float = 5.0):
        self.interval_s = interval_s
        self._t0 = time.monotonic()
        self._prompt = 0
        self._gen = 0
        self.last: Optional[StepStats] = None

    def record(self, stats: StepStats) -> None:
        self._prompt += stats.num_tokens - stats.num_generated
        self._gen += stats.num_generated
        self.last = stats
        now = time.monotonic()
        if now - self._t0 >= self.interval_s:
            dt = now - self._t0
            extra = ""
            if stats.prefix_cache_queries:
                extra += " | prefix cache hit rate %.1f%%" % (100.0 * stats.prefix_cache_hits / stats.prefix_cache_queries)
            if stats.num_draft_tokens:
                extra += " | draft acceptance %.1f%%" % (100.0 * stats.num_accepted_tokens / stats.num_draft_tokens)
            logger.info("throughput: prompt %.1f tok/s, generation %.1f tok/s | running %d, waiting %d | KV usage %.1f%%%s",
                        self._prompt / dt, self._gen / dt, stats.num_running, stats.num_waiting, 100 * stats.kv_usage,
                        extra)
            self._t0, self._prompt, self._gen = now, 0, 0


class PrometheusStatLogger:
    """Gauges / counters / histograms under the ``tokenweave:`` prefix (needs ``prometheus_client``)."""

    def __init__(self, model_name: str = ""):
        import prometheus_client as pc
        labels = {"model_name": model_name}
        reg = pc.CollectorRegistry()
        self.registry = reg
        self.running = pc.Gauge("tokenweave:num_requests_running", "running requests", list(labels), registry=reg).labels(**labels)
        self.waiting = pc.Gauge("tokenweave:num_requests_waiting", "waiting requests", list(labels), registry=reg).labels(**labels)
        self.kv_usage = pc.Gauge("tokenweave:kv_cache_usage", "fraction of KV blocks in use", list(labels), registry=reg).labels(**labels)
        self.prompt_tokens = pc.Counter("tokenweave:prompt_tokens_total", "prefill tokens", list(labels), registry=reg).labels(**labels)
        self.gen_tokens = pc.Counter("tokenweave:generation_tokens_total", "generated tokens", list(labels), registry=reg).labels(**labels)
        self.step_tokens = pc.Histogram("tokenweave:iteration_tokens", "tokens per step", list(labels), registry=reg,
                                        buckets=[1, 8, 64, 256, 1024, 2048, 4096, 8192, 16384, 32768, 65536]).labels(**labels)
        self.ttft = pc.Histogram("tokenweave:time_to_first_token_seconds", "TTFT", list(labels), registry=reg,
                                 buckets=[0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1, 2.5, 5, 10]).labels(**labels)
        self.e2e = pc.Histogram("tokenweave:e2e_request_latency_seconds", "request latency", list(labels), registry=reg,
                                buckets=[0.1, 0.5, 1, 2.5, 5, 10, 30, 60, 120]).labels(**labels)
        self.tpot = pc.Histogram("tokenweave:time_per_output_token_seconds", "mean time per output token after the first",
                                 list(labels), registry=reg,
                                 buckets=[0.005, 0.01, 0.02, 0.03, 0.05, 0.075, 0.1, 0.2, 0.5, 1]).labels(**labels)
        counter = lambda name, doc: pc.Counter(name, doc, list(labels), registry=reg).labels(**labels)  # noqa: E731
        self.prefix_queries = counter("tokenweave:prefix_cache_queries_total", "blocks looked up in the prefix cache")
        self.prefix_hits = counter("tokenweave:prefix_cache_hits_total", "blocks found in the prefix cache")
        self.draft_tokens = counter("tokenweave:spec_decode_num_draft_tokens_total", "draft tokens proposed")
        self.accepted_tokens = counter("tokenweave:spec_decode_num_accepted_tokens_total", "draft tokens confirmed")
        self._seen = [0, 0, 0, 0]       # last cumulative values, to turn them into increments

    def record(self, stats: StepStats) -> None:
        self.running.set(stats.num_running)
        self.waiting.set(stats.num_waiting)
        self.kv_usage.set(stats.kv_usage)
        self.prompt_tokens.inc(max(0, stats.num_tokens - stats.num_generated))
        self.gen_tokens.inc(stats.num_generated)
        self.step_tokens.observe(stats.num_tokens)
        now = [stats.prefix_cache_queries, stats.prefix_cache_hits, stats.num_draft_tokens, stats.num_accepted_tokens]
        for c, new, old in zip((self.prefix_queries, self.prefix_hits, self.draft_tokens, self.accepted_tokens),
                               now, self._seen):
            c.inc(max(0, new - old))
        self._seen = now

    def record_finished(self, ttft_s: Optional[float], e2e_s: Optional[float], tpot_s: Optional[float] = None) -> None:
        if ttft_s is not None:
            self.ttft.observe(ttft_s)
        if e2e_s is not None:
            self.e2e.observe(e2e_s)
        if tpot_s is not None:
            self.tpot.observe(tpot_s)
