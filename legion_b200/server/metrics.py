"""Prometheus metrics (``legion_*`` families, ``src/server/metrics.rs`` in the reference) and the log ring
behind ``/v1/logs/stream``."""
from __future__ import annotations

import logging
import threading
from collections import deque
from typing import List, Tuple

from prometheus_client import CollectorRegistry, Counter, Gauge, Histogram, generate_latest

_LAT = (0.005, 0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1, 2.5, 5, 10, 30, 60, 120)
_ITL = (0.001, 0.002, 0.005, 0.01, 0.02, 0.05, 0.1, 0.25, 0.5, 1)


class Metrics:
    def __init__(self):
        r = self.registry = CollectorRegistry()
        self.http_requests = Counter("legion_http_requests", "HTTP requests", ["path", "method", "status"], registry=r)
        self.request_latency = Histogram("legion_request_latency", "request latency (s)", ["path"], buckets=_LAT, registry=r)
        self.ttft = Histogram("legion_time_to_first_token", "time to first token (s)", buckets=_LAT, registry=r)
        self.itl = Histogram("legion_inter_token_latency", "inter-token latency (s)", buckets=_ITL, registry=r)
        self.prompt_tokens = Counter("legion_prompt_tokens", "prompt tokens processed", registry=r)
        self.completion_tokens = Counter("legion_completion_tokens", "tokens generated", registry=r)
        self.in_flight = Gauge("legion_requests_in_flight", "HTTP requests in flight", registry=r)
        g = lambda n, d: Gauge(f"legion_engine_{n}", d, registry=r)
        self.e_running = g("running", "sequences running")
        self.e_waiting = g("waiting", "requests waiting")
        self.e_waiting_keys = g("waiting_keys", "distinct fair-share keys waiting")
        self.e_kv_used = g("kv_blocks_used", "KV blocks in use")
        self.e_kv_total = g("kv_blocks_total", "KV blocks in the cache")
        self.e_preempt = g("kv_preemptions", "sequences preempted for KV space")
        self.e_prefix_hit = g("prefix_cache_hit_tokens", "prompt tokens served from the prefix cache")
        self.e_spec_draft = g("spec_draft_tokens", "draft tokens proposed")
        self.e_spec_acc = g("spec_accepted_tokens", "draft tokens accepted")
        self.e_spec_rate = g("spec_acceptance_rate", "accepted / drafted")
        self.e_spec_len = g("spec_mean_accepted_length", "tokens per verify step")
        self.e_spec_k = g("spec_mean_k", "mean draft length")
        self.e_spec_steps = g("spec_verify_steps", "verify steps")
        self.e_steps = g("steps", "engine steps")
        self.e_step_ms = g("step_ms", "engine step time, EWMA (ms)")
        self.e_model_bytes = g("model_bytes_step", "bytes a step must read (analytic)")
        self.e_waiting_prio = Gauge("legion_engine_waiting_by_priority", "requests waiting per priority", ["priority"],
                                    registry=r)
        self.gpu = {n: Gauge(f"legion_gpu_{n}", d, ["gpu"], registry=r) for n, d in (
            ("nvlink_rx_bytes", "NVLink bytes received"), ("nvlink_tx_bytes", "NVLink bytes sent"),
            ("pcie_rx_bytes", "PCIe bytes received"), ("pcie_tx_bytes", "PCIe bytes sent"),
            ("memory_busy_seconds", "memory controller busy time"), ("sm_busy_seconds", "SM busy time"))}

    def update_engine(self, st):
        self.e_running.set(st.running)
        self.e_waiting.set(st.waiting)
        self.e_waiting_keys.set(st.waiting_keys)
        self.e_kv_used.set(st.kv_blocks_used)
        self.e_kv_total.set(st.kv_blocks_total)
        self.e_preempt.set(st.kv_preemptions)
        self.e_prefix_hit.set(st.prefix_cache_hit_tokens)
        self.e_spec_draft.set(st.spec_draft_tokens)
        self.e_spec_acc.set(st.spec_accepted_tokens)
        self.e_spec_rate.set(st.spec_acceptance_rate)
        self.e_spec_len.set(st.spec_mean_accepted_length)
        self.e_spec_k.set(st.spec_mean_k)
        self.e_spec_steps.set(st.spec_verify_steps)
        self.e_steps.set(st.steps)
        self.e_step_ms.set(st.step_ms_ewma)
        self.e_model_bytes.set(st.model_bytes_step)
        for p, n in st.waiting_by_priority.items():
            self.e_waiting_prio.labels(priority=str(p)).set(n)

    def render(self) -> str:
        return generate_latest(self.registry).decode()


class LogRing(logging.Handler):
    """Last N log lines, readable incrementally."""

    def __init__(self, capacity: int = 2000):
        super().__init__()
        self._buf = deque(maxlen=capacity)
        self._n = 0
        self._lock = threading.Lock()
        self.setFormatter(logging.Formatter("%(asctime)s %(levelname)s %(name)s: %(message)s"))

    def emit(self, record):
        with self._lock:
            self._buf.append(self.format(record))
            self._n += 1

    def since(self, seen: int) -> Tuple[List[str], int]:
        with self._lock:
            new = self._n - seen
            if new <= 0:
                return [], self._n
            return list(self._buf)[-min(new, len(self._buf)):], self._n
