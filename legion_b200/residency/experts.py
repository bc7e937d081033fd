"""Expert residency: where routed-expert weights live and how the ones a step needs reach the GPU.

Modes (``--experts``, ``src/residency/mod.rs:206-246`` in the reference):
  device   every expert in HBM (default: 180 GB per GPU holds the benchmark models whole)
  cache    all experts in pinned host memory, ``n_slots`` of them cached in HBM slots per layer; a step first
           makes every expert it routes to resident (misses are copied into the coldest slots), then the
           grouped GEMM runs over the slot tensor through a remap table expert -> slot
  host     cache mode with the minimum number of slots (a step's experts only)
  ssd      cache mode whose backing store is a file per layer on disk (``--expert-dir``), read through a memory map,
           with a bounded tier of recently used experts in (pinned) host memory in between (``--expert-ram-gib``):
           HBM slots <- RAM tier <- file (``src/residency/ssd_experts.rs``, ``host_tier.rs`` in the reference)
  peer     experts sharded over the GPUs' symmetric memory; the grouped GEMM's TMA loads stream a peer's
           expert tiles over NVLink straight into the consumer's shared-memory ring (no staging copy, no
           cluster multicast): see ``PeerExperts``

Policy: decayed routing heat per expert (``src/residency/policy.rs``); the victim of a miss is the resident
expert with the lowest heat that the current step does not use. Hit / miss / byte counters feed the metrics.
The host-copy backing lets the whole mechanism run on the CPU for tests, as in the reference
(``src/residency/experts.rs:14-17``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch


@dataclass
class CacheStats:
    hits: int = 0
    misses: int = 0
    bytes_copied: int = 0
    steps: int = 0
    ram_hits: int = 0          # ssd mode: misses served from the RAM tier
    ssd_reads: int = 0         # ssd mode: misses read from the file
    ssd_bytes: int = 0

    @property
    def hit_rate(self) -> float:
        n = self.hits + self.misses
        return self.hits / n if n else 1.0


class ExpertCache:
    """One MoE layer's experts behind ``n_slots`` device slots."""

    def __init__(self, gate_up: torch.Tensor, down: torch.Tensor, n_slots: int, device, decay: float = 0.95,
                 profile: Optional[List[float]] = None, ssd_path: Optional[str] = None, ram_experts: int = 0):
        self.E = gate_up.shape[0]
        self.n_slots = min(n_slots, self.E)
        self.device = torch.device(device)
        pin = self.device.type == "cuda"
        self.ssd = None
        self.ram: "Dict[int, Tuple[torch.Tensor, torch.Tensor]]" = {}     # ssd mode: expert -> (gate_up, down), LRU order
        self.ram_experts = max(0, ram_experts)
        if ssd_path is not None:
            # the layer's experts as raw 16- or 32-bit words in one file: [E, gate_up words | down words]
            import numpy as np
            wt = {2: torch.int16, 4: torch.int32}[gate_up.element_size()]
            flat = torch.cat([gate_up.detach().cpu().contiguous().view(self.E, -1).view(wt),
                              down.detach().cpu().contiguous().view(self.E, -1).view(wt)], dim=1).contiguous()
            flat.numpy().tofile(ssd_path)
            self.ssd = np.memmap(ssd_path, dtype=flat.numpy().dtype, mode="r", shape=tuple(flat.shape))
            self._shape_gu, self._shape_dn = tuple(gate_up.shape[1:]), tuple(down.shape[1:])
            self._n_gu = gate_up[0].numel()
            self._dtype = gate_up.dtype
            self.host_gu = self.host_dn = None
            del flat
        else:
            self.host_gu = gate_up.detach().cpu().contiguous()
            self.host_dn = down.detach().cpu().contiguous()
            if pin:
                self.host_gu, self.host_dn = self.host_gu.pin_memory(), self.host_dn.pin_memory()
        self.slot_gu = torch.empty((self.n_slots,) + tuple(gate_up.shape[1:]), dtype=gate_up.dtype, device=self.device)
        self.slot_dn = torch.empty((self.n_slots,) + tuple(down.shape[1:]), dtype=down.dtype, device=self.device)
        self.slot_of = [-1] * self.E              # expert -> slot
        self.expert_in = [-1] * self.n_slots      # slot -> expert
        self.heat = list(profile) if profile else [0.0] * self.E
        self.decay = decay
        self.stats = CacheStats()
        self.bytes_per_expert = (gate_up[0].numel() + down[0].numel()) * gate_up.element_size()
        # seed the slots with the hottest experts of the profile (or the first ones)
        order = sorted(range(self.E), key=lambda e: -self.heat[e])[:self.n_slots]
        for s, e in enumerate(order):
            self._load(e, s)
        self.stats = CacheStats()
        # Device-side tables (GPU, experts in pinned host memory): decode-sized steps make their experts resident
        # inside ONE kernel launch (csrc/residency.cu) that reads the routing on the device, picks victims by the
        # same decayed heat, and copies misses straight from the mapped host memory, so such steps need no host
        # round trip and stay inside a CUDA graph. The device tables are then the authoritative ones; the host
        # policy (prompt-sized steps) reads them back first and uploads them again afterwards.
        self.dev = None
        self.device_rows = 64
        if pin and self.ssd is None and self.E <= 2048 and self.bytes_per_expert % 16 == 0:
            self._upload_tables()

    # ------------------------------------------------------------------ device-side tables
    def _upload_tables(self):
        """Host lists -> device tables (created once; captured graphs keep pointing at the same tensors)."""
        if self.dev is None:
            i32 = dict(dtype=torch.int32, device=self.device)
            self.dev = {"slot_of": torch.empty(self.E, **i32), "expert_in": torch.empty(self.n_slots, **i32),
                        "heat": torch.empty(self.E, dtype=torch.float32, device=self.device),
                        "miss": torch.zeros(2 * self.n_slots, **i32), "ctl": torch.zeros(4, **i32),
                        "stats": torch.zeros(4, dtype=torch.int64, device=self.device)}
        d = self.dev
        d["slot_of"].copy_(torch.tensor(self.slot_of, dtype=torch.int32))
        d["expert_in"].copy_(torch.tensor(self.expert_in, dtype=torch.int32))
        d["heat"].copy_(torch.tensor(self.heat, dtype=torch.float32))

    def _download_tables(self):
        d = self.dev
        self.slot_of = d["slot_of"].tolist()
        self.expert_in = d["expert_in"].tolist()
        self.heat = d["heat"].tolist()
        hits, misses, nbytes, steps = d["stats"].tolist()
        d["stats"].zero_()
        self.stats.hits += hits
        self.stats.misses += misses
        self.stats.bytes_copied += nbytes
        self.stats.steps += steps

    @property
    def graph_safe(self) -> bool:
        return self.dev is not None

    def prepare_on_device(self, ids: torch.Tensor) -> torch.Tensor:
        from ..ops import sm100
        d = self.dev
        out = torch.empty_like(ids)
        ws = sm100.Workspace.get(ids.device)
        sm100.ext().expert_cache_prepare(ids.contiguous(), d["slot_of"], d["expert_in"], d["heat"], self.decay,
                                         self.host_gu, self.host_dn, self.slot_gu, self.slot_dn, out, d["miss"],
                                         d["ctl"], d["stats"], ws.status)
        return out

    def sync_stats(self) -> CacheStats:
        """Counters including the steps that ran on the device (synchronises)."""
        if self.dev is not None:
            self._download_tables()
        return self.stats

    def _host_copy(self, e: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """The expert's weights in host memory: the resident copy, or (ssd mode) the RAM tier, filled from the file."""
        if self.ssd is None:
            return self.host_gu[e], self.host_dn[e]
        hit = self.ram.pop(e, None)
        if hit is not None:
            self.stats.ram_hits += 1
            self.ram[e] = hit                      # most recently used last
            return hit
        import numpy as np
        row = torch.from_numpy(np.array(self.ssd[e]))          # one sequential read of the expert's bytes
        self.stats.ssd_reads += 1
        self.stats.ssd_bytes += self.bytes_per_expert
        gu = row[:self._n_gu].view(self._dtype).view(self._shape_gu)
        dn = row[self._n_gu:].view(self._dtype).view(self._shape_dn)
        if self.device.type == "cuda":
            gu, dn = gu.pin_memory(), dn.pin_memory()
        if self.ram_experts > 0:
            while len(self.ram) >= self.ram_experts:
                self.ram.pop(next(iter(self.ram)))
            self.ram[e] = (gu, dn)
        return gu, dn

    def _load(self, e: int, s: int):
        old = self.expert_in[s]
        if old >= 0:
            self.slot_of[old] = -1
        gu, dn = self._host_copy(e)
        self.slot_gu[s].copy_(gu, non_blocking=self.ssd is None)
        self.slot_dn[s].copy_(dn, non_blocking=self.ssd is None)
        self.slot_of[e], self.expert_in[s] = s, e
        self.stats.bytes_copied += self.bytes_per_expert

    def prepare(self, ids: torch.Tensor) -> torch.Tensor:
        """Makes every expert in ``ids`` [T, k] resident and returns the same routing in slot numbers."""
        if self.dev is not None and ids.is_cuda and ids.shape[0] <= self.device_rows:
            return self.prepare_on_device(ids)
        if self.dev is not None:
            self._download_tables()             # the device tables are the authoritative ones
        need = sorted(set(ids.flatten().tolist()))
        if len(need) > self.n_slots:
            raise RuntimeError(f"a step routes to {len(need)} experts but the cache has {self.n_slots} slots; "
                               "lower the batch or raise --expert-cache-gib")
        for e in range(self.E):
            self.heat[e] *= self.decay
        using = set(need)
        for e in need:
            self.heat[e] += 1.0
            if self.slot_of[e] >= 0:
                self.stats.hits += 1
                continue
            self.stats.misses += 1
            victims = [s for s in range(self.n_slots) if self.expert_in[s] not in using]
            free = [s for s in victims if self.expert_in[s] < 0]
            s = free[0] if free else min(victims, key=lambda v: self.heat[self.expert_in[v]])
            self._load(e, s)
        self.stats.steps += 1
        if self.dev is not None:
            self._upload_tables()
            return self.dev["slot_of"][ids.long()].to(torch.int32)
        table = torch.tensor(self.slot_of, dtype=torch.int32, device=ids.device)
        return table[ids.long()].to(torch.int32)

    def weights(self) -> Tuple[torch.Tensor, torch.Tensor]:
        return self.slot_gu, self.slot_dn

    def profile(self) -> List[float]:
        return list(self.heat)


def slots_for_budget(cfg, gib: float, dtype_bytes: int = 2) -> int:
    """Slots per layer that fit ``gib`` GiB of HBM for the routed experts of all MoE layers."""
    per_expert = 3 * cfg.hidden * cfg.expert_ff * dtype_bytes
    n_moe = sum(1 for il in range(cfg.n_layer) if cfg.is_moe_layer(il))
    if n_moe == 0 or per_expert == 0:
        return 0
    return max(cfg.top_k, int(gib * (1 << 30) / (per_expert * n_moe)))


class PeerExperts:
    """Experts sharded over the ranks' symmetric memory. ``views(r)`` returns rank r's shard as tensors backed
    by the peer mapping; a grouped GEMM given such a tensor streams the weights over NVLink with plain
    (non-multicast) TMA loads, tile by tile, overlapped with the math of the tiles before it."""

    def __init__(self, gate_up_local: torch.Tensor, down_local: torch.Tensor, group, rank: int, world: int):
        from ..parallel.dist import no_multicast_default
        no_multicast_default()
        import torch.distributed._symmetric_memory as symm_mem
        self.rank, self.world = rank, world
        self.per = gate_up_local.shape[0]
        self.shape_gu, self.shape_dn = tuple(gate_up_local.shape), tuple(down_local.shape)
        n_gu, n_dn = gate_up_local.numel(), down_local.numel()
        self.buf = symm_mem.empty(n_gu + n_dn, dtype=gate_up_local.dtype, device=gate_up_local.device)
        self.buf[:n_gu].copy_(gate_up_local.reshape(-1))
        self.buf[n_gu:].copy_(down_local.reshape(-1))
        self.handle = symm_mem.rendezvous(self.buf, group=group)
        self._n_gu = n_gu
        torch.cuda.synchronize()
        import torch.distributed as dist
        dist.barrier(group=group)

    def views(self, r: int) -> Tuple[torch.Tensor, torch.Tensor]:
        if r == self.rank:
            flat = self.buf
        else:
            flat = self.handle.get_buffer(r, (self.buf.numel(),), self.buf.dtype)
        return flat[:self._n_gu].view(self.shape_gu), flat[self._n_gu:].view(self.shape_dn)

    def expert_range(self, r: int) -> Tuple[int, int]:
        return r * self.per, (r + 1) * self.per
