"""NUMA placement of a rank's host threads next to its GPU.

Pinned staging buffers, the packed step inputs and the loader's read buffers are touched by host threads every
step; on a two-socket host they should live on the socket the GPU hangs off. ``bind_to_gpu`` looks the GPU's PCI
device up in sysfs, reads its NUMA node and that node's CPU list, and restricts the calling process to those CPUs
(memory then follows first touch). Everything is read from sysfs; nothing on the GPU is changed. Reference
counterpart: the NUMA-local pinned inboxes and thread placement of ``src/hw`` / ``src/model/glm5next/par/exchange.rs``.
"""
from __future__ import annotations

import os
from typing import List, Optional


def parse_cpulist(text: str) -> List[int]:
    """'0-3,8,10-11' -> [0, 1, 2, 3, 8, 10, 11]"""
    cpus: List[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-", 1)
            cpus.extend(range(int(a), int(b) + 1))
        else:
            cpus.append(int(part))
    return cpus


def pci_bus_id(index: int) -> Optional[str]:
    """'0000:1b:00.0' of CUDA device ``index`` (lower case, the way sysfs spells it), or None."""
    try:
        import pynvml
        pynvml.nvmlInit()
        info = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(index))
        bus = info.busId.decode() if isinstance(info.busId, bytes) else info.busId
        bus = bus.lower()
        return bus[4:] if len(bus.split(":")[0]) == 8 else bus      # NVML pads the domain to 8 digits
    except Exception:
        return None


def gpu_numa_node(bus_id: str, sysfs: str = "/sys") -> Optional[int]:
    try:
        with open(os.path.join(sysfs, "bus/pci/devices", bus_id, "numa_node")) as f:
            node = int(f.read().strip())
        return node if node >= 0 else None
    except (OSError, ValueError):
        return None


def node_cpus(node: int, sysfs: str = "/sys") -> List[int]:
    try:
        with open(os.path.join(sysfs, "devices/system/node", f"node{node}", "cpulist")) as f:
            return parse_cpulist(f.read())
    except OSError:
        return []


def bind_to_gpu(index: int, sysfs: str = "/sys", bus_id: Optional[str] = None, apply=os.sched_setaffinity) -> dict:
    """Restricts this process to the CPUs of GPU ``index``'s NUMA node. Returns what was found and done; a host
    without NUMA information (one node, containers that hide sysfs) is left as it is."""
    bus = bus_id or pci_bus_id(index)
    out = {"gpu": index, "bus_id": bus, "node": None, "cpus": [], "bound": False}
    if bus is None:
        return out
    node = gpu_numa_node(bus, sysfs)
    out["node"] = node
    if node is None:
        return out
    cpus = node_cpus(node, sysfs)
    try:
        allowed = set(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        allowed = set(cpus)
    cpus = [c for c in cpus if c in allowed]
    out["cpus"] = cpus
    if cpus:
        try:
            apply(0, set(cpus))
            out["bound"] = True
        except OSError:
            pass
    return out
