"""Prometheus text exposition with the reference's metric names and labels.

Parity: `crates/saber-serve/src/metrics.rs:1-8` (families `saber:num_requests_running/waiting`,
`saber:prompt_tokens_total`, `saber:generation_tokens_total`, `saber:time_to_first_token_seconds`,
`saber:inter_token_latency_seconds`, `saber:step_time_seconds`, `saber:e2e_request_latency_seconds`,
`saber:request_queue_time_seconds`, `saber:spec_decode_*`, `saber:request_success/refused_total`),
fixed-bucket histograms with PromQL-style quantiles (`hist.rs:1-15`), and the "which path" census
counters mirrored on /metrics (`census.rs:1-25`).
"""
from __future__ import annotations

import threading
from bisect import bisect_left

BUCKETS = (0.001, 0.0025, 0.005, 0.0075, 0.01, 0.015, 0.02, 0.025, 0.03, 0.04, 0.05, 0.075, 0.1, 0.15,
           0.2, 0.3, 0.5, 0.75, 1.0, 2.5, 5.0, 10.0, 30.0, 60.0)


class Histogram:
    def __init__(self, buckets=BUCKETS):
        self.buckets = tuple(buckets)
        self.counts = [0] * (len(self.buckets) + 1)
        self.sum = 0.0
        self.n = 0

    def observe(self, v: float) -> None:
        self.counts[bisect_left(self.buckets, v)] += 1
        self.sum += v
        self.n += 1

    def quantile(self, q: float) -> float:
        """histogram_quantile semantics: linear interpolation inside the bucket."""
        if self.n == 0:
            return 0.0
        rank, acc = q * self.n, 0
        for i, c in enumerate(self.counts):
            if acc + c >= rank and c > 0:
                lo = self.buckets[i - 1] if i > 0 else 0.0
                hi = self.buckets[i] if i < len(self.buckets) else self.buckets[-1]
                return lo + (hi - lo) * (rank - acc) / c
            acc += c
        return self.buckets[-1]

    def render(self, name: str, labels: str) -> list:
        out, acc = [], 0
        for b, c in zip(self.buckets, self.counts):
            acc += c
            out.append(f'{name}_bucket{{{labels},le="{b}"}} {acc}')
        out.append(f'{name}_bucket{{{labels},le="+Inf"}} {self.n}')
        out.append(f"{name}_sum{{{labels}}} {self.sum}")
        out.append(f"{name}_count{{{labels}}} {self.n}")
        return out


class Metrics:
    HISTS = ("time_to_first_token_seconds", "inter_token_latency_seconds", "step_time_seconds",
             "e2e_request_latency_seconds", "request_queue_time_seconds")

    def __init__(self, model_name: str = "saber"):
        self.labels = f'engine="0",model_name="{model_name}"'
        self.h = {k: Histogram() for k in self.HISTS}
        self.counters = {"request_success_total": 0, "request_refused_total": 0, "image_requests_total": 0}
        self._lock = threading.Lock()

    def observe(self, name: str, v: float) -> None:
        with self._lock:
            self.h[name].observe(v)

    def inc(self, name: str, n: int = 1) -> None:
        with self._lock:
            self.counters[name] = self.counters.get(name, 0) + n

    def render(self, engine_stats: dict, census: dict = None) -> str:
        L = self.labels
        lines = []
        def gauge(name, v, help_=""):
            lines.append(f"# TYPE saber:{name} gauge")
            lines.append(f"saber:{name}{{{L}}} {v}")
        def counter(name, v):
            lines.append(f"# TYPE saber:{name} counter")
            lines.append(f"saber:{name}{{{L}}} {v}")
        gauge("num_requests_running", engine_stats.get("running", 0))
        gauge("num_requests_waiting", engine_stats.get("waiting", 0))
        gauge("kv_cache_usage_perc", 1.0 - engine_stats.get("kv_free_blocks", 0) / max(1, engine_stats.get("kv_total_blocks", 1)))
        counter("prompt_tokens_total", engine_stats.get("prompt_tokens", 0))
        counter("generation_tokens_total", engine_stats.get("generation_tokens", 0))
        counter("spec_decode_num_drafts_total", engine_stats.get("drafts", 0))
        counter("spec_decode_num_draft_tokens_total", engine_stats.get("draft_tokens", 0))
        counter("spec_decode_num_accepted_tokens_total", engine_stats.get("accepted_tokens", 0))
        lines.append("# TYPE saber:spec_decode_num_accepted_tokens_per_pos_total counter")
        for pos, v in enumerate(engine_stats.get("accepted_per_pos", [])):
            lines.append(f'saber:spec_decode_num_accepted_tokens_per_pos_total{{{L},position="{pos}"}} {v}')
        counter("prefix_cache_queries_total", engine_stats.get("prefix_lookups", 0))
        counter("prefix_cache_hits_total", engine_stats.get("prefix_hits", 0))
        counter("prefix_cache_hit_tokens_total", engine_stats.get("prefix_hit_tokens", 0))
        with self._lock:
            for k, v in self.counters.items():
                counter(k, v)
            for k, hst in self.h.items():
                lines.append(f"# TYPE saber:{k} histogram")
                lines += hst.render(f"saber:{k}", L)
        for k, v in (census or {}).items():
            lines.append(f"# TYPE saber_census_{k} counter")
            lines.append(f"saber_census_{k}{{{L}}} {v}")
        return "\n".join(lines) + "\n"
