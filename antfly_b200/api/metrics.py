"""Prometheus metrics (names keep the reference's ``antfly_inference_`` prefix: zig/pkg/inference/src/server/
metrics.zig:24-63): request counters and latency per endpoint, queue depth, scheduler and KV gauges."""
from __future__ import annotations

from prometheus_client import CollectorRegistry, Counter, Gauge, Histogram, generate_latest


class Metrics:
    def __init__(self):
        self.registry = CollectorRegistry()
        r = self.registry
        self.requests = Counter("antfly_inference_requests_total", "Requests by endpoint and status",
                                ["endpoint", "status"], registry=r)
        self.latency = Histogram("antfly_inference_request_seconds", "Request latency", ["endpoint"], registry=r)
        self.tokens = Counter("antfly_inference_tokens_total", "Tokens processed", ["endpoint", "kind"], registry=r)
        self.cache = Counter("antfly_inference_result_cache_total", "Result-cache lookups by endpoint and outcome",
                             ["endpoint", "outcome"], registry=r)
        self.queue_depth = Gauge("antfly_inference_queue_depth", "Requests waiting for a slot", registry=r)
        self.queue_rejected = Counter("antfly_inference_queue_rejected_total", "Requests refused with 503", registry=r)
        self.loaded_models = Gauge("antfly_inference_loaded_models", "Models resident in GPU memory", registry=r)
        self.sched = Gauge("antfly_inference_scheduler", "Scheduler counters", ["counter"], registry=r)
        self.kv_free_blocks = Gauge("antfly_inference_kv_free_blocks", "Free KV-cache blocks", ["model"], registry=r)
        self.spec = Gauge("antfly_inference_speculative", "Speculative decoding counters", ["counter"], registry=r)
        self.kernel_launches = Gauge("antfly_inference_kernel_launches_total", "CUDA kernel launches issued",
                                     registry=r)

    def render(self) -> bytes:
        return generate_latest(self.registry)
