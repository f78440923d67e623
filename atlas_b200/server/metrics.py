"""Prometheus metrics (``/metrics``).

Reference parity: ``crates/spark-server/src/metrics.rs`` (``atlas_requests_total``, ``atlas_requests_active``,
``atlas_time_to_first_token_seconds{model}``, ``atlas_generation_tokens_total``, HTTP byte counters),
``scheduler/port_gauges.rs``, prefix-cache hit counters of ``spark-runtime/src/prefix_cache.rs:24-50``.
"""
from __future__ import annotations

from typing import Optional

from prometheus_client import CollectorRegistry, Counter, Gauge, Histogram, generate_latest


class ServerMetrics:
    def __init__(self, model: str):
        self.model = model
        r = self.registry = CollectorRegistry()
        self.requests_total = Counter("atlas_requests_total", "Finished generation requests", ["model"], registry=r)
        self.http_total = Counter("atlas_http_requests_total", "HTTP requests", ["path", "status"], registry=r)
        self.http_bytes_in = Counter("atlas_http_request_bytes_total", "HTTP request body bytes", registry=r)
        self.http_latency = Histogram("atlas_http_request_seconds", "HTTP request latency", ["path"], registry=r)
        self.ttft = Histogram("atlas_time_to_first_token_seconds", "Time to first token", ["model"], registry=r,
                              buckets=(.005, .01, .025, .05, .1, .25, .5, 1, 2.5, 5, 10, 30))
        self.gen_tokens = Counter("atlas_generation_tokens_total", "Generated tokens", ["model"], registry=r)
        self.prompt_tokens = Counter("atlas_prompt_tokens_total", "Prompt tokens", ["model"], registry=r)
        self.active = Gauge("atlas_requests_active", "Requests being processed", registry=r)
        self.waiting = Gauge("atlas_requests_waiting", "Requests queued", registry=r)
        self.kv_free = Gauge("atlas_kv_blocks_free", "Free KV blocks", registry=r)
        self.kv_total = Gauge("atlas_kv_blocks_total", "Total KV blocks", registry=r)
        self.decoded = Gauge("atlas_decoded_tokens_total", "Tokens emitted by the scheduler", registry=r)
        self.tps = Gauge("atlas_delivered_tokens_per_second", "Recent delivered tokens per second", registry=r)
        self.preempt = Gauge("atlas_preemptions_total", "Sequences preempted", registry=r)
        self.prefix_hits = Gauge("atlas_prefix_cache_hits_total", "Prefix-cache lookups that hit", registry=r)
        self.prefix_lookups = Gauge("atlas_prefix_cache_lookups_total", "Prefix-cache lookups", registry=r)
        self.prefix_hit_tokens = Gauge("atlas_prefix_cache_hit_tokens_total", "Prompt tokens served from cache", registry=r)
        self.spec_proposed = Gauge("atlas_spec_proposed_tokens_total", "Draft tokens proposed", registry=r)
        self.spec_accepted = Gauge("atlas_spec_accepted_tokens_total", "Draft tokens accepted", registry=r)
        self.gpu_fault = Gauge("atlas_gpu_fault", "1 once the GPU context is lost", registry=r)
        self.conf_mean_top1 = Histogram("atlas_confidence_mean_top1", "Mean top-1 probability over a request's first tokens",
                                        registry=r, buckets=(.1, .2, .3, .4, .5, .6, .7, .8, .9, .95, 1.0))
        self.conf_min_margin = Histogram("atlas_confidence_min_margin", "Smallest top-1 / top-2 probability gap of a request",
                                         registry=r, buckets=(.01, .02, .05, .1, .2, .3, .5, .7, 1.0))
        self.conf_low_frac = Histogram("atlas_confidence_low_fraction", "Fraction of a request's first tokens with top-1 < 0.5",
                                       registry=r, buckets=(0, .05, .1, .2, .3, .5, .7, 1.0))

    def on_confidence(self, summary) -> None:
        if summary:
            self.conf_mean_top1.observe(summary["mean_top1"])
            self.conf_min_margin.observe(summary["min_margin"])
            self.conf_low_frac.observe(summary["low_frac"])

    def on_http(self, path: str, status: int, seconds: float, bytes_in: int) -> None:
        p = path if len(path) < 48 else path[:48]
        self.http_total.labels(p, str(status)).inc()
        self.http_latency.labels(p).observe(seconds)
        if bytes_in:
            self.http_bytes_in.inc(bytes_in)

    def on_request_done(self, prompt_tokens: int, completion_tokens: int, ttft_s: Optional[float]) -> None:
        self.requests_total.labels(self.model).inc()
        self.gen_tokens.labels(self.model).inc(completion_tokens)
        self.prompt_tokens.labels(self.model).inc(prompt_tokens)
        if ttft_s is not None:
            self.ttft.labels(self.model).observe(ttft_s)

    def observe_engine(self, engine) -> None:
        from ..utils.fault import FAULT_LATCH
        s = engine.snapshot()
        self.active.set(s["running"] + s["prefilling"])
        self.waiting.set(s["waiting"])
        self.kv_free.set(s["kv_free_blocks"])
        self.kv_total.set(s["kv_total_blocks"])
        self.decoded.set(s["generation_tokens"])
        self.tps.set(s["tokens_per_s"])
        self.preempt.set(s["preemptions"])
        self.prefix_hits.set(s.get("prefix_hits", 0))
        self.prefix_lookups.set(s.get("prefix_lookups", 0))
        self.prefix_hit_tokens.set(s.get("prefix_hit_tokens", 0))
        self.spec_proposed.set(s["spec_proposed"])
        self.spec_accepted.set(s["spec_accepted"])
        self.gpu_fault.set(1 if FAULT_LATCH.tripped else 0)

    def render(self) -> str:
        return generate_latest(self.registry).decode()
