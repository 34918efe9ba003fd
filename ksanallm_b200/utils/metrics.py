"""Metrics registry with the reference's metric names, exposed three ways: Prometheus text at ``GET /metrics``,
periodic OTLP/HTTP JSON export when ``setting.profiler.metrics_export_url`` is an http(s) URL, and stdout when it
is ``debug``. Reference: src/ksana_llm/profiler/profiler.cpp:40-130 (REPORT_METRIC / REPORT_COUNTER) and the
catalogue in docs/monitoring_metrics_guide.md:18-120.
"""
from __future__ import annotations

import json
import threading
import time
from typing import Any, Dict, List, Optional

_BUCKETS_US = [1e3, 2e3, 5e3, 1e4, 2e4, 5e4, 1e5, 2e5, 5e5, 1e6, 2e6, 5e6, 1e7, 3e7, 6e7]


class Histogram:
    def __init__(self, name: str, buckets=None):
        self.name = name
        self.buckets = list(buckets or _BUCKETS_US)
        self.counts = [0] * (len(self.buckets) + 1)
        self.sum = 0.0
        self.n = 0
        self.lock = threading.Lock()

    def observe(self, v: float) -> None:
        with self.lock:
            self.sum += v
            self.n += 1
            for i, b in enumerate(self.buckets):
                if v <= b:
                    self.counts[i] += 1
                    return
            self.counts[-1] += 1


class Metrics:
    HISTOGRAMS = ["time_to_first_token_us", "inter_token_interval_latency_us", "total_latency_us",
                  "input_tokens_len", "output_token_len", "forward_req_total_latency_us", "batch_scheduler_time_us",
                  "forward_time_us", "sampling_time_us", "time_per_output_token_us"]
    COUNTERS = ["forward_req_total_num", "forward_req_error_num", "forward_req_timeout_num", "forward_req_aborted_num",
                "forward_req_exceed_capacity_num", "generated_token_num", "prefix_cache_hit_token_num",
                "prefix_cache_hit_req_num", "swap_out_block_num", "swap_in_block_num", "recompute_req_num",
                "spec_draft_token_num", "spec_accepted_token_num"]
    GAUGES = ["batch_scheduler_waiting_req_num", "batch_scheduler_running_req_num", "batch_scheduler_swapped_req_num",
              "block_manager_free_block_num", "block_manager_used_block_num", "block_manager_usage_ratio",
              "global_token_throughput", "local_token_throughput"]

    def __init__(self, export_url: str = "", interval_ms: int = 60000, timeout_ms: int = 1000,
                 attributes: Optional[Dict[str, Any]] = None):
        self.h = {n: Histogram(n) for n in self.HISTOGRAMS}
        self.c = {n: 0 for n in self.COUNTERS}
        self.g = {n: 0.0 for n in self.GAUGES}
        self.lock = threading.Lock()
        self.export_url = export_url or ""
        self.interval = max(interval_ms, 100) / 1000.0
        self.timeout = max(timeout_ms, 100) / 1000.0
        self.attributes = dict(attributes or {})
        self._stop = threading.Event()
        self._thread = None
        self._last_tokens = 0
        self._last_time = time.time()
        if self.export_url:
            self._thread = threading.Thread(target=self._export_loop, daemon=True, name="ksana-metrics-export")
            self._thread.start()

    @classmethod
    def from_serving_config(cls, serving) -> "Metrics":
        p = serving.setting.profiler
        return cls(p.metrics_export_url, p.export_interval_millis, p.export_timeout_millis, p.attributes)

    def report_metric(self, name: str, value: float) -> None:
        h = self.h.get(name)
        if h is None:
            h = self.h[name] = Histogram(name)
        h.observe(float(value))

    def report_counter(self, name: str, inc: int = 1) -> None:
        with self.lock:
            self.c[name] = self.c.get(name, 0) + inc

    def set_gauge(self, name: str, value: float) -> None:
        self.g[name] = float(value)

    # ---- engine hooks ---------------------------------------------------------------------------------------
    def observe_request(self, req) -> None:
        self.report_counter("forward_req_total_num")
        if req.error is not None:
            self.report_counter("forward_req_error_num")
        n_out = sum(len(s.output_tokens) for s in req.seqs)
        self.report_counter("generated_token_num", n_out)
        self.report_metric("input_tokens_len", len(req.prompt_tokens))
        self.report_metric("output_token_len", n_out)
        if req.first_token_time is not None:
            self.report_metric("time_to_first_token_us", (req.first_token_time - req.arrival) * 1e6)
        if req.finish_time is not None:
            self.report_metric("total_latency_us", (req.finish_time - req.arrival) * 1e6)
        tt = req.token_times
        if len(tt) > 1:
            self.report_metric("time_per_output_token_us", (tt[-1] - tt[0]) / (len(tt) - 1) * 1e6)
            for a, b in zip(tt[:-1], tt[1:]):
                if b > a:
                    self.report_metric("inter_token_interval_latency_us", (b - a) * 1e6)

    def refresh_from_engine(self, llm) -> None:
        self.set_gauge("batch_scheduler_waiting_req_num", llm.sched.num_waiting)
        self.set_gauge("batch_scheduler_running_req_num", llm.sched.num_running)
        self.set_gauge("batch_scheduler_swapped_req_num", llm.sched.num_swapped)
        free = llm.cache.num_available_blocks
        total = llm.cache.num_device_blocks
        self.set_gauge("block_manager_free_block_num", free)
        self.set_gauge("block_manager_used_block_num", total - free)
        self.set_gauge("block_manager_usage_ratio", (total - free) / max(total, 1))
        now = time.time()
        toks = llm.stats["generated_tokens"]
        dt = max(now - self._last_time, 1e-6)
        self.set_gauge("global_token_throughput", (toks - self._last_tokens) / dt)
        self.set_gauge("local_token_throughput", (toks - self._last_tokens) / dt)
        self._last_tokens, self._last_time = toks, now
        st, cs = llm.sched.stats, llm.cache.stats
        with self.lock:
            self.c["prefix_cache_hit_token_num"] = cs.prefix_hit_tokens
            self.c["swap_out_block_num"] = cs.swapped_out_blocks
            self.c["swap_in_block_num"] = cs.swapped_in_blocks
            self.c["recompute_req_num"] = st.preempt_recompute
            self.c["spec_draft_token_num"] = st.draft_proposed
            self.c["spec_accepted_token_num"] = st.draft_accepted
            self.c["forward_req_timeout_num"] = st.timeouts
            self.c["flexible_cache_hit_token_num"] = cs.flexible_hit_tokens
            self.c["pp_micro_batch_migration_num"] = st.mb_migrations
            self.g["spec_draft_hit_rate"] = st.draft_accepted / st.draft_proposed if st.draft_proposed else 0.0

    # ---- exposition --------------------------------------------------------------------------------------------
    def prometheus_text(self) -> str:
        out: List[str] = []
        for n, v in self.c.items():
            out += [f"# TYPE ksana_{n} counter", f"ksana_{n} {v}"]
        for n, v in self.g.items():
            out += [f"# TYPE ksana_{n} gauge", f"ksana_{n} {v}"]
        for n, h in self.h.items():
            out.append(f"# TYPE ksana_{n} histogram")
            acc = 0
            for b, c in zip(h.buckets, h.counts):
                acc += c
                out.append(f'ksana_{n}_bucket{{le="{b:g}"}} {acc}')
            out.append(f'ksana_{n}_bucket{{le="+Inf"}} {h.n}')
            out += [f"ksana_{n}_sum {h.sum}", f"ksana_{n}_count {h.n}"]
        return "\n".join(out) + "\n"

    def otlp_json(self) -> Dict[str, Any]:
        now = int(time.time() * 1e9)
        metrics = []
        for n, v in self.c.items():
            metrics.append({"name": n, "sum": {"aggregationTemporality": 2, "isMonotonic": True,
                                               "dataPoints": [{"asInt": str(int(v)), "timeUnixNano": str(now)}]}})
        for n, v in self.g.items():
            metrics.append({"name": n, "gauge": {"dataPoints": [{"asDouble": v, "timeUnixNano": str(now)}]}})
        for n, h in self.h.items():
            metrics.append({"name": n, "histogram": {"aggregationTemporality": 2, "dataPoints": [{
                "count": str(h.n), "sum": h.sum, "bucketCounts": [str(c) for c in h.counts],
                "explicitBounds": h.buckets, "timeUnixNano": str(now)}]}})
        attrs = [{"key": k, "value": {"stringValue": str(v)}} for k, v in self.attributes.items()]
        return {"resourceMetrics": [{"resource": {"attributes": attrs},
                                     "scopeMetrics": [{"scope": {"name": "ksanallm_b200"}, "metrics": metrics}]}]}

    def _export_loop(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                if self.export_url == "debug":
                    print(json.dumps(self.otlp_json())[:2000], flush=True)
                elif self.export_url.startswith("http"):
                    import urllib.request
                    req = urllib.request.Request(self.export_url, data=json.dumps(self.otlp_json()).encode(),
                                                 headers={"Content-Type": "application/json"})
                    urllib.request.urlopen(req, timeout=self.timeout).read()
            except Exception:
                pass

    def close(self) -> None:
        self._stop.set()


def add_metrics_route(app, metrics: Metrics, llm) -> None:
    from fastapi.responses import PlainTextResponse

    @app.get("/metrics")
    async def _metrics():
        metrics.refresh_from_engine(llm)
        return PlainTextResponse(metrics.prometheus_text())
