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
            ("memory_busy_seconds", "memory controller busy time"), ("sm_busy_seconds", "SM busy time"),
            ("sm_clock_mhz", "SM clock"), ("power_watts", "board power"), ("memory_used_bytes", "HBM in use"))}
        # per-stage host time of the engine step (plan / build / forward / finish), accumulated
        self.e_host_ms = Gauge("legion_engine_host_ms", "host time per step phase, accumulated (ms)", ["phase"], registry=r)
        # KV / prefix-cache tiers
        self.e_swap_out = g("kv_swap_out", "preempted sequences parked in host memory")
        self.e_swap_in = g("kv_swap_in", "parked sequences copied back")
        self.e_prefix_lookup = g("prefix_cache_lookup_tokens", "prompt tokens looked up in the prefix cache")
        self.e_prefix_spill = g("prefix_host_spilled", "prefix-cache blocks spilled to the host tier")
        self.e_prefix_restore = g("prefix_host_restored", "prefix-cache blocks restored from the host tier")
        # rooflines: the measured peaks of this machine and where the running engine sits against them
        rf = lambda n, d: Gauge(f"legion_roofline_{n}", d, registry=r)
        self.r_hbm = rf("hbm_gbs", "measured copy bandwidth (GB/s)")
        self.r_bf16 = rf("bf16_tflops", "measured cuBLAS bf16 throughput (TFLOP/s)")
        self.r_nvlink = rf("nvlink_gbs_per_direction", "measured peer-copy bandwidth per direction (GB/s)")
        self.r_step_floor = rf("step_floor_ms", "bytes a decode step must read / measured copy bandwidth (ms)")
        self.r_step_frac = rf("step_bandwidth_fraction", "step floor / measured step time")
        # tensor-parallel communication of this rank
        self.tp_reductions = Gauge("legion_tp_all_reduce_calls", "all-reduce calls of this rank", registry=r)
        self.tp_bytes = Gauge("legion_tp_all_reduce_bytes", "bytes reduced by this rank", registry=r)
        self._busy = {}

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
        for phase, ms in (st.host_ms or {}).items():
            self.e_host_ms.labels(phase=phase).set(ms)
        self.e_swap_out.set(st.kv_swap_out)
        self.e_swap_in.set(st.kv_swap_in)
        self.e_prefix_lookup.set(st.prefix_cache_lookup_tokens)
        self.e_prefix_spill.set(st.prefix_host_spilled)
        self.e_prefix_restore.set(st.prefix_host_restored)
        self.update_roofline(st)

    def update_roofline(self, st, peaks=None):
        """Measured peaks and the step's distance from the copy-bandwidth floor."""
        if peaks is None:
            from ..hw.gpu import NVLINK_GBS_PER_DIR, measured_peaks
            peaks = dict(measured_peaks(), nvlink_gbs=NVLINK_GBS_PER_DIR)
        self.r_hbm.set(peaks["hbm_gbs"])
        self.r_bf16.set(peaks["bf16_tflops"])
        self.r_nvlink.set(peaks.get("nvlink_gbs", 0.0))
        floor_ms = st.model_bytes_step / (peaks["hbm_gbs"] * 1e9) * 1e3 if st.model_bytes_step else 0.0
        self.r_step_floor.set(floor_ms)
        self.r_step_frac.set(floor_ms / st.step_ms_ewma if st.step_ms_ewma > 0 else 0.0)

    def update_parallel(self, stats: dict):
        """``ParallelCtx.stats`` of this rank."""
        self.tp_reductions.set(stats.get("all_reduce", 0))
        self.tp_bytes.set(stats.get("bytes", 0))

    def sample_gpus(self, nvml=None, now=None):
        """Reads (never writes) NVML: NVLink and PCIe byte counters, utilisation integrated into busy seconds, clocks,
        power and memory of every visible GPU. ``nvml``: the pynvml module (a fake in tests); absent NVML leaves the
        gauges at zero."""
        import time
        if nvml is None:
            try:
                import pynvml as nvml
                nvml.nvmlInit()
            except Exception:
                return 0
        now = time.monotonic() if now is None else now
        n = 0
        try:
            count = nvml.nvmlDeviceGetCount()
        except Exception:
            return 0
        for i in range(count):
            try:
                h = nvml.nvmlDeviceGetHandleByIndex(i)
            except Exception:
                continue
            lab = str(i)

            def put(name, fn):
                try:
                    self.gpu[name].labels(gpu=lab).set(fn())
                except Exception:
                    pass
            # NVLink throughput counters are cumulative KiB per device (field values, summed over the links)
            def nvlink(field):
                vals = nvml.nvmlDeviceGetFieldValues(h, [field])
                return float(vals[0].value.ullVal) * 1024.0
            if hasattr(nvml, "NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_RX"):
                put("nvlink_rx_bytes", lambda: nvlink(nvml.NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_RX))
                put("nvlink_tx_bytes", lambda: nvlink(nvml.NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_TX))
            put("pcie_rx_bytes", lambda: nvml.nvmlDeviceGetPcieThroughput(h, nvml.NVML_PCIE_UTIL_RX_BYTES) * 1024.0)
            put("pcie_tx_bytes", lambda: nvml.nvmlDeviceGetPcieThroughput(h, nvml.NVML_PCIE_UTIL_TX_BYTES) * 1024.0)
            put("sm_clock_mhz", lambda: nvml.nvmlDeviceGetClockInfo(h, nvml.NVML_CLOCK_SM))
            put("power_watts", lambda: nvml.nvmlDeviceGetPowerUsage(h) / 1000.0)
            put("memory_used_bytes", lambda: nvml.nvmlDeviceGetMemoryInfo(h).used)
            try:
                u = nvml.nvmlDeviceGetUtilizationRates(h)
                last, sm_s, mem_s = self._busy.get(i, (now, 0.0, 0.0))
                dt = max(0.0, now - last)
                sm_s += dt * u.gpu / 100.0
                mem_s += dt * u.memory / 100.0
                self._busy[i] = (now, sm_s, mem_s)
                self.gpu["sm_busy_seconds"].labels(gpu=lab).set(sm_s)
                self.gpu["memory_busy_seconds"].labels(gpu=lab).set(mem_s)
            except Exception:
                pass
            n += 1
        return n

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
