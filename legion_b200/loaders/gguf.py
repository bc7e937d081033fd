"""GGUF v3 reader and writer (own implementation of the file format, memory-mapped tensor data) and
block de-quantisation for F32 / F16 / BF16 / Q8_0 / Q4_0 / Q4_1 / Q5_0 / Q5_1 / Q4_K / Q5_K / Q6_K / IQ4_NL.

The reference reads GGUF through ggml's ``gguf_*`` API (``src/gguf.rs:23-660``) and leaves quantised blocks
to ggml's kernels; here quantised tensors are expanded to the compute dtype at load time.
Split files ``name-00001-of-0000N.gguf`` are discovered and merged (``src/gguf/split.rs``).
"""
from __future__ import annotations

import mmap
import os
import re
import struct
from dataclasses import dataclass
from typing import Any, BinaryIO, Dict, List, Optional, Tuple

import numpy as np

MAGIC = b"GGUF"
(T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64) = range(13)
_SCALAR = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f", T_BOOL: "<?",
           T_U64: "<Q", T_I64: "<q", T_F64: "<d"}

# ggml tensor types: id -> (name, block elements, block bytes)
GGML_TYPES = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22),
    7: ("Q5_1", 32, 24), 8: ("Q8_0", 32, 34), 10: ("Q2_K", 256, 84), 11: ("Q3_K", 256, 110), 12: ("Q4_K", 256, 144),
    13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210), 15: ("Q8_K", 256, 292), 20: ("IQ4_NL", 32, 18),
    24: ("I8", 1, 1), 25: ("I16", 1, 2), 26: ("I32", 1, 4), 27: ("I64", 1, 8), 28: ("F64", 1, 8), 30: ("BF16", 1, 2),
}
TYPE_ID = {v[0]: k for k, v in GGML_TYPES.items()}


@dataclass
class TensorInfo:
    name: str
    shape: Tuple[int, ...]      # numpy order (slowest first) = reversed ggml ne[]
    ggml_type: int
    offset: int                 # relative to the data section
    file_index: int = 0

    @property
    def type_name(self) -> str:
        return GGML_TYPES[self.ggml_type][0]

    @property
    def n_elements(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def n_bytes(self) -> int:
        _, be, bb = GGML_TYPES[self.ggml_type]
        return self.n_elements // be * bb


class _Reader:
    def __init__(self, buf):
        self.b, self.p = buf, 0

    def read(self, fmt):
        v = struct.unpack_from(fmt, self.b, self.p)[0]
        self.p += struct.calcsize(fmt)
        return v

    def string(self) -> str:
        n = self.read("<Q")
        s = bytes(self.b[self.p:self.p + n]).decode("utf-8", "replace")
        self.p += n
        return s

    def value(self, t):
        if t in _SCALAR:
            return self.read(_SCALAR[t])
        if t == T_STR:
            return self.string()
        if t == T_ARR:
            et = self.read("<I")
            n = self.read("<Q")
            if et in _SCALAR and et != T_BOOL:
                fmt = _SCALAR[et]
                sz = struct.calcsize(fmt)
                arr = np.frombuffer(self.b, dtype=np.dtype(fmt), count=n, offset=self.p)
                self.p += sz * n
                return arr.tolist()
            return [self.value(et) for _ in range(n)]
        raise ValueError(f"unknown GGUF value type {t}")


class GgufFile:
    """One GGUF model (possibly split over several files)."""

    def __init__(self, path: str):
        self.paths = discover_splits(path)
        self.metadata: Dict[str, Any] = {}
        self.tensors: Dict[str, TensorInfo] = {}
        self._maps: List[mmap.mmap] = []
        self._data_start: List[int] = []
        for fi, p in enumerate(self.paths):
            f = open(p, "rb")
            mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            f.close()
            self._maps.append(mm)
            r = _Reader(mm)
            if bytes(mm[:4]) != MAGIC:
                raise ValueError(f"{p}: not a GGUF file")
            r.p = 4
            version = r.read("<I")
            if version not in (2, 3):
                raise ValueError(f"{p}: unsupported GGUF version {version}")
            n_tensors, n_kv = r.read("<Q"), r.read("<Q")
            md = {}
            for _ in range(n_kv):
                k = r.string()
                t = r.read("<I")
                md[k] = r.value(t)
            if fi == 0:
                self.metadata = md
            else:
                for k, v in md.items():
                    self.metadata.setdefault(k, v)
            infos = []
            for _ in range(n_tensors):
                name = r.string()
                nd = r.read("<I")
                ne = [r.read("<Q") for _ in range(nd)]
                tt = r.read("<I")
                off = r.read("<Q")
                infos.append(TensorInfo(name, tuple(reversed(ne)), tt, off, fi))
            align = int(md.get("general.alignment", 32))
            self._data_start.append((r.p + align - 1) // align * align)
            for ti in infos:
                self.tensors[ti.name] = ti

    @property
    def arch(self) -> str:
        return self.metadata.get("general.architecture", "")

    def raw(self, name: str) -> np.ndarray:
        ti = self.tensors[name]
        start = self._data_start[ti.file_index] + ti.offset
        return np.frombuffer(self._maps[ti.file_index], dtype=np.uint8, count=ti.n_bytes, offset=start)

    def numpy(self, name: str) -> np.ndarray:
        """Tensor as float32 (or its integer type), de-quantised if needed, in numpy (row-major) shape."""
        ti = self.tensors[name]
        return dequantize(self.raw(name), ti.ggml_type, ti.shape)

    DEVICE_TYPES = {2, 8, 12, 13, 14, 20}       # block formats with a device de-quantisation kernel

    def torch(self, name: str, dtype=None, device=None):
        """``device``: a CUDA device moves the raw block bytes there and expands them to bf16 with the
        ``gguf_dequant`` kernel (the host never touches the elements); other tensors go through numpy."""
        import torch
        ti = self.tensors[name]
        raw = self.raw(name)
        if device is not None and torch.device(device).type == "cuda" and ti.ggml_type in self.DEVICE_TYPES:
            from ..ops.sm100 import ext
            dev_raw = torch.from_numpy(np.array(raw, copy=True)).to(device, non_blocking=True)
            out = torch.empty(ti.shape, dtype=torch.bfloat16, device=device)
            ext().gguf_dequant(dev_raw, ti.ggml_type, out)
            return out.to(dtype) if dtype is not None else out
        if ti.type_name == "BF16":
            t = torch.frombuffer(bytearray(raw.tobytes()), dtype=torch.bfloat16).view(ti.shape)
        else:
            t = torch.from_numpy(np.ascontiguousarray(self.numpy(name)))
        return t.to(dtype) if dtype is not None else t

    def close(self):
        for m in self._maps:
            m.close()
        self._maps = []


def discover_splits(path: str) -> List[str]:
    m = re.match(r"^(.*)-(\d{5})-of-(\d{5})\.gguf$", path)
    if not m:
        return [path]
    base, n = m.group(1), int(m.group(3))
    return [f"{base}-{i:05d}-of-{n:05d}.gguf" for i in range(1, n + 1)]


# ----------------------------------------------------------------------------------------------------
# de-quantisation (vectorised over blocks)
# ----------------------------------------------------------------------------------------------------
def _f16(b: np.ndarray) -> np.ndarray:
    return b.view(np.float16).astype(np.float32)


def _scale_min_k4(sc: np.ndarray):
    """sc: [n, 12] uint8 -> (scales [n, 8], mins [n, 8]) 6-bit values."""
    d = np.empty(sc.shape[:-1] + (8,), dtype=np.uint8)
    m = np.empty_like(d)
    d[..., :4] = sc[..., 0:4] & 63
    m[..., :4] = sc[..., 4:8] & 63
    d[..., 4:] = (sc[..., 8:12] & 0xF) | ((sc[..., 0:4] >> 6) << 4)
    m[..., 4:] = (sc[..., 8:12] >> 4) | ((sc[..., 4:8] >> 6) << 4)
    return d.astype(np.float32), m.astype(np.float32)


_IQ4NL = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.float32)


def dequantize(raw: np.ndarray, ggml_type: int, shape: Tuple[int, ...]) -> np.ndarray:
    name, be, bb = GGML_TYPES[ggml_type]
    if name == "F32":
        return raw.view(np.float32).reshape(shape)
    if name == "F16":
        return raw.view(np.float16).astype(np.float32).reshape(shape)
    if name == "BF16":
        u = raw.view(np.uint16).astype(np.uint32) << 16
        return u.view(np.float32).reshape(shape)
    if name in ("I8", "I16", "I32", "I64", "F64"):
        return raw.view({"I8": np.int8, "I16": np.int16, "I32": np.int32, "I64": np.int64, "F64": np.float64}[name]).reshape(shape)
    blk = raw.reshape(-1, bb)
    n = blk.shape[0]
    if name == "Q8_0":
        d = _f16(blk[:, 0:2].copy())
        q = blk[:, 2:].view(np.int8).astype(np.float32)
        out = q * d
    elif name == "Q4_0":
        d = _f16(blk[:, 0:2].copy())
        qs = blk[:, 2:]
        out = np.concatenate([(qs & 0xF).astype(np.float32) - 8, (qs >> 4).astype(np.float32) - 8], axis=1) * d
    elif name == "Q4_1":
        d, m = _f16(blk[:, 0:2].copy()), _f16(blk[:, 2:4].copy())
        qs = blk[:, 4:]
        out = np.concatenate([(qs & 0xF).astype(np.float32), (qs >> 4).astype(np.float32)], axis=1) * d + m
    elif name in ("Q5_0", "Q5_1"):
        o = 2 if name == "Q5_0" else 4
        d = _f16(blk[:, 0:2].copy())
        qh = blk[:, o:o + 4].copy().view(np.uint32)          # [n, 1]
        qs = blk[:, o + 4:]
        j = np.arange(16, dtype=np.uint32)
        h0 = ((qh >> j) & 1).astype(np.uint8) << 4
        h1 = ((qh >> (j + 16)) & 1).astype(np.uint8) << 4
        q = np.concatenate([(qs & 0xF) | h0, (qs >> 4) | h1], axis=1).astype(np.float32)
        if name == "Q5_0":
            out = (q - 16) * d
        else:
            out = q * d + _f16(blk[:, 2:4].copy())
    elif name == "IQ4_NL":
        d = _f16(blk[:, 0:2].copy())
        qs = blk[:, 2:]
        out = np.concatenate([_IQ4NL[qs & 0xF], _IQ4NL[qs >> 4]], axis=1) * d
    elif name == "Q4_K":
        d, dmin = _f16(blk[:, 0:2].copy()), _f16(blk[:, 2:4].copy())
        sc, mn = _scale_min_k4(blk[:, 4:16])
        qs = blk[:, 16:144].reshape(n, 4, 32)
        lo = (qs & 0xF).astype(np.float32)
        hi = (qs >> 4).astype(np.float32)
        q = np.stack([lo, hi], axis=2).reshape(n, 8, 32)        # sub-block 2i = low nibbles, 2i+1 = high
        out = (q * (d * sc)[:, :, None] - (dmin * mn)[:, :, None]).reshape(n, 256)
    elif name == "Q5_K":
        d, dmin = _f16(blk[:, 0:2].copy()), _f16(blk[:, 2:4].copy())
        sc, mn = _scale_min_k4(blk[:, 4:16])
        qh = blk[:, 16:48]                                       # [n, 32]
        qs = blk[:, 48:176].reshape(n, 4, 32)
        i = np.arange(4, dtype=np.uint8)
        b1 = ((qh[:, None, :] >> (2 * i)[None, :, None]) & 1).astype(np.float32) * 16
        b2 = ((qh[:, None, :] >> (2 * i + 1)[None, :, None]) & 1).astype(np.float32) * 16
        lo = (qs & 0xF).astype(np.float32) + b1
        hi = (qs >> 4).astype(np.float32) + b2
        q = np.stack([lo, hi], axis=2).reshape(n, 8, 32)
        out = (q * (d * sc)[:, :, None] - (dmin * mn)[:, :, None]).reshape(n, 256)
    elif name == "Q6_K":
        ql = blk[:, 0:128].reshape(n, 2, 64)
        qh = blk[:, 128:192].reshape(n, 2, 32)
        sc = blk[:, 192:208].view(np.int8).astype(np.float32).reshape(n, 2, 8)
        d = _f16(blk[:, 208:210].copy())
        l0, l1 = ql[:, :, :32], ql[:, :, 32:]
        q1 = ((l0 & 0xF) | ((qh & 3) << 4)).astype(np.int8) - 32
        q2 = ((l1 & 0xF) | (((qh >> 2) & 3) << 4)).astype(np.int8) - 32
        q3 = ((l0 >> 4) | (((qh >> 4) & 3) << 4)).astype(np.int8) - 32
        q4 = ((l1 >> 4) | (((qh >> 6) & 3) << 4)).astype(np.int8) - 32
        q = np.stack([q1, q2, q3, q4], axis=2).astype(np.float32)      # [n, 2, 4, 32]
        # scale index for element l of quarter j: j * 2 + l // 16
        s = sc.reshape(n, 2, 4, 2)
        out = (q.reshape(n, 2, 4, 2, 16) * s[..., None]).reshape(n, 256) * d
    elif name == "Q2_K":
        # 16 groups of 16: a 4-bit scale and a 4-bit minimum each; 2-bit values, four per byte, the four bit pairs
        # of a 32-byte run giving four consecutive groups of 32
        scb = blk[:, 0:16]
        qs = blk[:, 16:80].reshape(n, 2, 1, 32)
        d, dmin = _f16(blk[:, 80:82].copy()), _f16(blk[:, 82:84].copy())
        shifts = np.array([0, 2, 4, 6], dtype=np.uint8).reshape(1, 1, 4, 1)
        q = ((qs >> shifts) & 3).astype(np.float32).reshape(n, 16, 16)         # [n, half, pair, 32] -> groups of 16
        sc = (scb & 0xF).astype(np.float32)
        mn = (scb >> 4).astype(np.float32)
        out = (q * (d * sc)[:, :, None] - (dmin * mn)[:, :, None]).reshape(n, 256)
    elif name == "Q3_K":
        # 2 low bits as in Q2_K plus a high bit from the mask bytes (bit j of byte l for the j-th group of 32;
        # a clear bit subtracts 4); 16 six-bit scales, offset by 32, packed into 12 bytes
        hm = blk[:, 0:32]
        qs = blk[:, 32:96].reshape(n, 2, 1, 32)
        a = blk[:, 96:108].copy().view(np.uint32).reshape(n, 3)
        d = _f16(blk[:, 108:110].copy())
        k1, k2 = np.uint32(0x03030303), np.uint32(0x0F0F0F0F)
        a0, a1, tmp = a[:, 0], a[:, 1], a[:, 2]
        aux = np.stack([(a0 & k2) | ((tmp & k1) << 4), (a1 & k2) | (((tmp >> 2) & k1) << 4),
                        ((a0 >> 4) & k2) | (((tmp >> 4) & k1) << 4), ((a1 >> 4) & k2) | (((tmp >> 6) & k1) << 4)], axis=1)
        sc = np.ascontiguousarray(aux).view(np.int8).reshape(n, 16).astype(np.float32) - 32.0
        shifts = np.array([0, 2, 4, 6], dtype=np.uint8).reshape(1, 1, 4, 1)
        low = ((qs >> shifts) & 3).astype(np.int16)                              # [n, 2, 4, 32]
        bits = np.arange(8, dtype=np.uint8).reshape(1, 8, 1)
        high = ((hm[:, None, :] >> bits) & 1).astype(np.int16).reshape(n, 2, 4, 32)
        q = (low - 4 * (1 - high)).astype(np.float32).reshape(n, 16, 16)
        out = (q * (d * sc)[:, :, None]).reshape(n, 256)
    else:
        raise NotImplementedError(f"GGUF tensor type {name} is not supported")
    return out.astype(np.float32).reshape(shape)


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """float32 [.., k] with k % 32 == 0 -> raw Q8_0 bytes."""
    b = x.astype(np.float32).reshape(-1, 32)
    amax = np.abs(b).max(axis=1, keepdims=True)
    d = amax / 127.0
    inv = np.where(d > 0, 1.0 / np.where(d > 0, d, 1), 0)
    q = np.rint(b * inv).astype(np.int8)
    out = np.empty((b.shape[0], 34), dtype=np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    b = x.astype(np.float32).reshape(-1, 32)
    idx = np.abs(b).argmax(axis=1)
    mx = b[np.arange(b.shape[0]), idx]
    d = mx / -8.0
    inv = np.where(d != 0, 1.0 / np.where(d != 0, d, 1), 0)
    q = np.clip(np.floor(b * inv[:, None] + 8.5), 0, 15).astype(np.uint8)
    out = np.empty((b.shape[0], 18), dtype=np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


# ----------------------------------------------------------------------------------------------------
# writer
# ----------------------------------------------------------------------------------------------------
class GgufWriter:
    def __init__(self, path: str, arch: str, alignment: int = 32):
        self.path, self.align = path, alignment
        self.kv: List[Tuple[str, int, Any]] = []
        self.tensors: List[Tuple[str, Tuple[int, ...], int, bytes]] = []
        self.add("general.architecture", arch)
        self.add("general.alignment", alignment, T_U32)

    def add(self, key: str, value: Any, vtype: Optional[int] = None):
        if vtype is None:
            if isinstance(value, bool):
                vtype = T_BOOL
            elif isinstance(value, int):
                vtype = T_U32 if 0 <= value < 2 ** 32 else T_I64
            elif isinstance(value, float):
                vtype = T_F32
            elif isinstance(value, str):
                vtype = T_STR
            elif isinstance(value, (list, tuple)):
                vtype = T_ARR
            else:
                raise TypeError(f"cannot infer the GGUF type of {key}")
        self.kv.append((key, vtype, value))

    def add_tensor(self, name: str, array, ggml_type: Optional[str] = None):
        """array: numpy float32 / float16 / int32, or a torch tensor (bfloat16 kept as BF16)."""
        raw_type = None
        try:
            import torch
            if isinstance(array, torch.Tensor):
                if array.dtype == torch.bfloat16 and ggml_type in (None, "BF16"):
                    shape = tuple(array.shape)
                    data = array.contiguous().view(torch.int16).numpy().tobytes()
                    self.tensors.append((name, shape, TYPE_ID["BF16"], data))
                    return
                array = array.detach().float().cpu().numpy()
        except ImportError:
            pass
        arr = np.ascontiguousarray(array)
        shape = tuple(arr.shape)
        if ggml_type in (None, "F32") and arr.dtype in (np.float32, np.float64):
            raw_type, data = "F32", arr.astype(np.float32).tobytes()
        elif ggml_type == "F16" or (ggml_type is None and arr.dtype == np.float16):
            raw_type, data = "F16", arr.astype(np.float16).tobytes()
        elif ggml_type == "BF16":
            u = arr.astype(np.float32).view(np.uint32)
            u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
            raw_type, data = "BF16", u.tobytes()
        elif ggml_type == "Q8_0":
            raw_type, data = "Q8_0", quantize_q8_0(arr).tobytes()
        elif ggml_type == "Q4_0":
            raw_type, data = "Q4_0", quantize_q4_0(arr).tobytes()
        elif arr.dtype == np.int32:
            raw_type, data = "I32", arr.tobytes()
        else:
            raise NotImplementedError(f"cannot write {arr.dtype} as {ggml_type}")
        self.tensors.append((name, shape, TYPE_ID[raw_type], data))

    @staticmethod
    def _str(s: str) -> bytes:
        b = s.encode("utf-8")
        return struct.pack("<Q", len(b)) + b

    def _value(self, t: int, v: Any) -> bytes:
        if t in _SCALAR:
            return struct.pack(_SCALAR[t], v)
        if t == T_STR:
            return self._str(v)
        if t == T_ARR:
            if len(v) == 0:
                return struct.pack("<IQ", T_I32, 0)
            e = v[0]
            et = T_STR if isinstance(e, str) else (T_F32 if isinstance(e, float) else (T_BOOL if isinstance(e, bool) else T_I32))
            out = [struct.pack("<IQ", et, len(v))]
            if et == T_STR:
                out.extend(self._str(x) for x in v)
            else:
                out.append(np.asarray(v, dtype=np.dtype(_SCALAR[et])).tobytes())
            return b"".join(out)
        raise ValueError(t)

    def write(self):
        head = [MAGIC, struct.pack("<IQQ", 3, len(self.tensors), len(self.kv))]
        for k, t, v in self.kv:
            head.append(self._str(k))
            head.append(struct.pack("<I", t))
            head.append(self._value(t, v))
        off = 0
        offsets = []
        for name, shape, tt, data in self.tensors:
            offsets.append(off)
            off = (off + len(data) + self.align - 1) // self.align * self.align
        for (name, shape, tt, data), o in zip(self.tensors, offsets):
            head.append(self._str(name))
            head.append(struct.pack("<I", len(shape)))
            head.append(b"".join(struct.pack("<Q", d) for d in reversed(shape)))
            head.append(struct.pack("<IQ", tt, o))
        blob = b"".join(head)
        pad = (-len(blob)) % self.align
        with open(self.path, "wb") as f:
            f.write(blob)
            f.write(b"\0" * pad)
            for (name, shape, tt, data), o in zip(self.tensors, offsets):
                f.write(data)
                f.write(b"\0" * ((-len(data)) % self.align))
