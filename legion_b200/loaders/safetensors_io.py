"""Safetensors files and HF checkpoint directories: memory-mapped reader, sharded index, writer, and
detection of the quantisation method (none / fp8 per-tensor / fp8 per-channel / fp8 128x128 blocks /
NVFP4 ModelOpt / NVFP4 compressed-tensors).

File format: 8-byte little-endian header length, JSON header {name: {dtype, shape, data_offsets}}, data.
Reference counterpart: ``src/safetensors.rs:154-711``.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Optional, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I64": torch.int64,
    "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
    "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        f = open(path, "rb")
        self._mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        f.close()
        (n,) = struct.unpack_from("<Q", self._mm, 0)
        if n > len(self._mm) - 8:
            raise ValueError(f"{path}: header length {n} exceeds the file size")
        self.header = json.loads(bytes(self._mm[8:8 + n]))
        self.metadata = self.header.pop("__metadata__", {})
        self._base = 8 + n

    def keys(self) -> List[str]:
        return list(self.header.keys())

    def info(self, name: str) -> Tuple[str, Tuple[int, ...]]:
        h = self.header[name]
        return h["dtype"], tuple(h["shape"])

    def span(self, name: str) -> Tuple[int, int]:
        """(absolute file offset, byte length) of a tensor's data."""
        a, b = self.header[name]["data_offsets"]
        return self._base + a, b - a

    def tensor(self, name: str) -> torch.Tensor:
        h = self.header[name]
        a, b = h["data_offsets"]
        dt = _DTYPES[h["dtype"]]
        if b == a:
            return torch.empty(h["shape"], dtype=dt)
        buf = memoryview(self._mm)[self._base + a:self._base + b]
        t = torch.frombuffer(buf, dtype=torch.uint8).clone() if dt in (torch.float8_e4m3fn, torch.float8_e5m2) \
            else torch.frombuffer(buf, dtype=dt)
        if dt in (torch.float8_e4m3fn, torch.float8_e5m2):
            t = t.view(dt)
        return t.view(h["shape"])


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None):
    header = {}
    if metadata:
        header["__metadata__"] = metadata
    off = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((-len(hj)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


class Checkpoint:
    """An HF checkpoint directory (or a single .safetensors file): tensor lookup across shards."""

    def __init__(self, path: str):
        self.dir = path if os.path.isdir(path) else os.path.dirname(path)
        self.files: Dict[str, SafetensorsFile] = {}
        self.where: Dict[str, str] = {}
        if os.path.isdir(path):
            idx = os.path.join(path, "model.safetensors.index.json")
            if os.path.exists(idx):
                wm = json.load(open(idx))["weight_map"]
                for name, fn in wm.items():
                    self.where[name] = fn
            else:
                for fn in sorted(os.listdir(path)):
                    if fn.endswith(".safetensors"):
                        for name in self._open(fn).keys():
                            self.where[name] = fn
        else:
            fn = os.path.basename(path)
            for name in self._open(fn).keys():
                self.where[name] = fn
        cfgp = os.path.join(self.dir, "config.json")
        self.config = json.load(open(cfgp)) if os.path.exists(cfgp) else {}

    def _open(self, fn: str) -> SafetensorsFile:
        f = self.files.get(fn)
        if f is None:
            f = SafetensorsFile(os.path.join(self.dir, fn))
            self.files[fn] = f
        return f

    def has(self, name: str) -> bool:
        return name in self.where

    def names(self) -> Iterable[str]:
        return self.where.keys()

    def get(self, name: str) -> torch.Tensor:
        t = self._ahead.pop(name, None) if self._ahead else None
        if t is not None:
            return t
        return self._open(self.where[name]).tensor(name)

    _ahead: Dict[str, torch.Tensor] = {}

    def prefetch(self, names: Iterable[str], threads: int = 8, chunk: int = 32 << 20, pin: bool = False) -> int:
        """Reads the data of ``names`` with a pool of ``threads`` positional reads (``os.preadv`` straight into the
        destination buffers, pieces of ``chunk`` bytes so that one large tensor is read by several threads at once)
        instead of faulting the memory map in page by page on the loading thread; the next ``get`` of each name
        returns the buffer that was read. ``pin``: page-locked buffers, for loads that go on to a GPU. Returns the
        bytes read. The reference's sharded parallel reader is ``src/load_io.rs:1-236``."""
        from concurrent.futures import ThreadPoolExecutor
        if self._ahead is Checkpoint._ahead:
            self._ahead = {}
        jobs = []
        fds: Dict[str, int] = {}
        total = 0
        for name in names:
            if name not in self.where or name in self._ahead:
                continue
            fn = self.where[name]
            f = self._open(fn)
            off, n = f.span(name)
            dtype_name, shape = f.info(name)
            raw = torch.empty(n, dtype=torch.uint8, pin_memory=bool(pin and n and torch.cuda.is_available()))
            self._ahead[name] = raw.view(_DTYPES[dtype_name]).view(shape) if n else torch.empty(shape, dtype=_DTYPES[dtype_name])
            if n == 0:
                continue
            if fn not in fds:
                fds[fn] = os.open(f.path, os.O_RDONLY)
            mv = memoryview(raw.numpy())
            for o in range(0, n, chunk):
                jobs.append((fds[fn], mv[o:min(n, o + chunk)], off + o))
            total += n

        def read(job):
            fd, buf, pos = job
            done = 0
            while done < len(buf):
                got = os.preadv(fd, [buf[done:]], pos + done)
                if got <= 0:
                    raise IOError("short read from a checkpoint file")
                done += got

        try:
            if jobs:
                with ThreadPoolExecutor(max_workers=max(1, threads)) as ex:
                    list(ex.map(read, jobs))
        finally:
            for fd in fds.values():
                os.close(fd)
        return total

    def quant_method(self) -> str:
        """none | fp8 | fp8_block | nvfp4 | nvfp4_ct"""
        qc = self.config.get("quantization_config") or {}
        method = (qc.get("quant_method") or "").lower()
        if method == "fp8":
            return "fp8_block" if qc.get("weight_block_size") else "fp8"
        if method == "modelopt":
            algo = (qc.get("quant_algo") or "").upper()
            return "nvfp4" if "NVFP4" in algo or "FP4" in algo else "fp8"
        if method == "compressed-tensors":
            fmt = json.dumps(qc).lower()
            return "nvfp4_ct" if "nvfp4" in fmt or '"num_bits": 4' in fmt else "fp8"
        hq = os.path.join(self.dir, "hf_quant_config.json")
        if os.path.exists(hq):
            algo = (json.load(open(hq)).get("quantization", {}).get("quant_algo") or "").upper()
            if "NVFP4" in algo:
                return "nvfp4"
            if "FP8" in algo:
                return "fp8"
        names = list(self.where.keys())
        if any(n.endswith(".weight_packed") for n in names):
            return "nvfp4_ct"
        if any(n.endswith(".weight_scale_2") for n in names):
            return "nvfp4"
        if any(n.endswith(".weight_scale_inv") for n in names):
            return "fp8_block"
        if any(n.endswith(".weight_scale") for n in names):
            return "fp8"
        return "none"
