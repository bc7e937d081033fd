"""Hardware discovery and measured rooflines: GPUs through NVML (read-only queries), NVLink presence, the
measured peaks file, and an analytic "model bytes" account of what a decode step must read.

Reference: ``src/hw/*.rs`` (NVML discovery, roofline table ``src/hw/roofline.rs:23-39``), ``src/ggml/model_bytes.rs``.
Nothing here changes a GPU setting: clocks, power limits, persistence and compute modes are only read.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

# measured on this pool when the peaks file is absent (copy bandwidth GB/s, cuBLAS bf16 TFLOP/s)
FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
NVLINK_GBS_PER_DIR = 770.0      # measured peer copy, per direction per GPU


def measured_peaks() -> dict:
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return dict(FALLBACK)


def gpus() -> List[dict]:
    out: List[dict] = []
    try:
        import pynvml
        pynvml.nvmlInit()
        for i in range(pynvml.nvmlDeviceGetCount()):
            h = pynvml.nvmlDeviceGetHandleByIndex(i)
            mem = pynvml.nvmlDeviceGetMemoryInfo(h)
            name = pynvml.nvmlDeviceGetName(h)
            d = {"index": i, "name": name.decode() if isinstance(name, bytes) else name,
                 "memory_total_mib": mem.total >> 20, "memory_used_mib": mem.used >> 20}
            try:
                d["sm_clock_mhz"] = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
                d["sm_clock_max_mhz"] = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
                d["power_w"] = pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0
                major, minor = pynvml.nvmlDeviceGetCudaComputeCapability(h)
                d["compute_capability"] = f"{major}.{minor}"
            except Exception:
                pass
            try:
                links = 0
                for l in range(18):
                    try:
                        if pynvml.nvmlDeviceGetNvLinkState(h, l):
                            links += 1
                    except Exception:
                        break
                d["nvlink_links"] = links
            except Exception:
                pass
            out.append(d)
    except Exception:
        pass
    return out


def nvml_counters(index: int = 0) -> Dict[str, float]:
    """NVLink / PCIe byte counters and utilisation for the metrics endpoint (best effort)."""
    out: Dict[str, float] = {}
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        try:
            out["pcie_tx_bytes"] = pynvml.nvmlDeviceGetPcieThroughput(h, pynvml.NVML_PCIE_UTIL_TX_BYTES) * 1024.0
            out["pcie_rx_bytes"] = pynvml.nvmlDeviceGetPcieThroughput(h, pynvml.NVML_PCIE_UTIL_RX_BYTES) * 1024.0
        except Exception:
            pass
        try:
            u = pynvml.nvmlDeviceGetUtilizationRates(h)
            out["sm_busy"] = u.gpu / 100.0
            out["memory_busy"] = u.memory / 100.0
        except Exception:
            pass
    except Exception:
        pass
    return out


def binary_arch_ok() -> Optional[str]:
    """The extension is built for sm_100a only; returns a message when the visible GPU is something else."""
    try:
        import torch
        if not torch.cuda.is_available():
            return None
        cc = torch.cuda.get_device_capability(0)
        return None if cc == (10, 0) else f"kernels are built for sm_100a, device 0 is sm_{cc[0]}{cc[1]}"
    except Exception:
        return None


def model_bytes_per_step(cfg, n_seqs: int, ctx: int, tp: int = 1, dtype_bytes: int = 2) -> dict:
    """Bytes one decode step of ``n_seqs`` sequences at context ``ctx`` must read from HBM on one rank:
    dense weights, the expected set of routed experts, and KV; divided by the measured copy bandwidth it is
    the step-time floor the bandwidth gauges compare against."""
    H = cfg.hidden
    dense = 0
    experts = 0
    kv = 0
    for il, kind in enumerate(cfg.layer_kinds):
        if kind in ("attn", "swa", "nope"):
            qw = cfg.n_head * cfg.head_dim * (2 if cfg.gated_attn else 1)
            dense += (qw + 2 * cfg.n_kv_head * cfg.head_dim) * H + H * cfg.n_head * cfg.head_dim
            kv += 2 * cfg.n_kv_head * cfg.head_dim * ctx * n_seqs
        elif kind == "gdn":
            dense += (cfg.gdn_conv_channels() + cfg.gdn_v_heads * cfg.gdn_v_dim * 2 + 2 * cfg.gdn_v_heads) * H
            kv += cfg.gdn_v_heads * cfg.gdn_k_dim * cfg.gdn_v_dim * 2 * n_seqs     # fp32 state read + write
        elif kind == "mla":
            dense += (cfg.q_lora + cfg.kv_lora + cfg.qk_rope_dim) * H + cfg.n_head * (cfg.qk_nope_dim + cfg.qk_rope_dim) * max(cfg.q_lora, 1)
            dense += cfg.n_head * (cfg.qk_nope_dim + cfg.v_head_dim) * cfg.kv_lora + H * cfg.n_head * cfg.v_head_dim
            kv += (cfg.kv_lora + cfg.qk_rope_dim) * ctx * n_seqs
        if cfg.is_moe_layer(il):
            E, k = cfg.n_expert, cfg.top_k
            active = E * (1.0 - (1.0 - k / E) ** n_seqs)
            experts += active * 3 * H * cfg.expert_ff
            dense += E * H + 3 * H * cfg.shared_ff
        elif cfg.dense_ff:
            dense += 3 * H * cfg.dense_ff
    head = cfg.vocab * H
    total = (dense / tp + experts / tp + head / tp + kv / tp) * dtype_bytes
    peaks = measured_peaks()
    return {"dense_bytes": dense * dtype_bytes / tp, "expert_bytes": experts * dtype_bytes / tp,
            "kv_bytes": kv * dtype_bytes / tp, "head_bytes": head * dtype_bytes / tp, "total_bytes": total,
            "floor_ms": total / (peaks["hbm_gbs"] * 1e9) * 1e3, "peaks": peaks["source"]}


def system_report() -> dict:
    import platform
    rep = {"python": platform.python_version(), "platform": platform.platform(), "gpus": gpus(),
           "measured_peaks": measured_peaks(), "nvlink_gbs_per_direction": NVLINK_GBS_PER_DIR}
    try:
        import torch
        rep["torch"] = torch.__version__
        rep["cuda_available"] = torch.cuda.is_available()
        if torch.cuda.is_available():
            rep["device_count"] = torch.cuda.device_count()
    except Exception:
        pass
    msg = binary_arch_ok()
    if msg:
        rep["warning"] = msg
    try:
        from ..ops import sm100
        rep["extension_loaded"] = sm100.have_ext()
    except Exception:
        rep["extension_loaded"] = False
    try:
        rep["numa_nodes"] = len([d for d in os.listdir("/sys/devices/system/node") if d.startswith("node")])
    except Exception:
        pass
    return rep
