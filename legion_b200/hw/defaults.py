"""Defaults that depend on the hardware: the sizes an engine starts with when the command line leaves them open.

The reference keys its defaults on the machine it finds (GPU generation and memory, unified-memory boxes, host
cores: ``src/hardware.rs``, ``src/cli/serve/defaults.rs``). Here the table is short because there is one target, but
the choice is still made from what the device reports, not hard-wired: a B200-class part (about 180 GB) takes
8192-token prompt chunks and 64-token pages; smaller parts step down so that
activations of a prompt chunk and the CUDA-graph buckets stay a small share of memory; CPU engines (tests, the
reference forward pass) use small chunks and 16-token pages."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class EngineDefaults:
    profile: str
    max_batch_tokens: int
    prefill_chunk: int
    kv_block: int
    max_seqs: int
    gpu_memory_utilization: float
    cuda_graphs: bool
    pipeline_micro: int


_CPU = EngineDefaults("cpu", 1024, 512, 16, 16, 0.0, False, 512)
_TABLE = [
    # (minimum device memory in GiB, defaults)
    (150.0, EngineDefaults("b200", 8192, 8192, 64, 16, 0.92, True, 2048)),
    (70.0, EngineDefaults("80g", 8192, 4096, 64, 16, 0.90, True, 2048)),
    (30.0, EngineDefaults("40g", 4096, 2048, 64, 8, 0.90, True, 1024)),
    (0.0, EngineDefaults("small", 2048, 1024, 32, 4, 0.85, True, 512)),
]


def engine_defaults(device: str = "cpu", total_gib: Optional[float] = None) -> EngineDefaults:
    """Defaults for an engine on ``device`` (``cpu`` | ``cuda[:N]``). ``total_gib`` overrides the memory the device
    reports (tests; a process that was given a share of a GPU)."""
    if not str(device).startswith("cuda"):
        return _CPU
    if total_gib is None:
        try:
            import torch
            idx = int(str(device).split(":")[1]) if ":" in str(device) else torch.cuda.current_device()
            total_gib = torch.cuda.get_device_properties(idx).total_memory / 2 ** 30
        except Exception:
            total_gib = 0.0
    for floor, d in _TABLE:
        if total_gib >= floor:
            return d
    return _TABLE[-1][1]
