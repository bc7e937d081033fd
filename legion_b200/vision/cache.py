"""Encoded image rows kept by image hash, least recently used first out, bounded in bytes (the reference keeps
256 MiB of them: ``src/vision/mod.rs`` row cache). A conversation re-sends its images with every turn; the tower
runs once per image."""
from __future__ import annotations

import hashlib
import threading
from collections import OrderedDict
from typing import Optional

import torch


def image_hash(data: bytes) -> bytes:
    return hashlib.sha256(data).digest()


class RowCache:
    def __init__(self, max_bytes: int = 256 << 20):
        self.max_bytes = max_bytes
        self._rows: "OrderedDict[bytes, object]" = OrderedDict()
        self._bytes = 0
        self._lock = threading.Lock()
        self.hits = 0
        self.misses = 0

    @staticmethod
    def _size(v) -> int:
        ts = v if isinstance(v, (list, tuple)) else [v]
        return sum(t.numel() * t.element_size() for t in _flatten(ts))

    def get(self, key: bytes):
        with self._lock:
            v = self._rows.get(key)
            if v is None:
                self.misses += 1
                return None
            self._rows.move_to_end(key)
            self.hits += 1
            return v

    def put(self, key: bytes, value) -> None:
        n = self._size(value)
        if n > self.max_bytes:
            return
        with self._lock:
            old = self._rows.pop(key, None)
            if old is not None:
                self._bytes -= self._size(old)
            self._rows[key] = value
            self._bytes += n
            while self._bytes > self.max_bytes and self._rows:
                _, ev = self._rows.popitem(last=False)
                self._bytes -= self._size(ev)

    @property
    def bytes(self) -> int:
        return self._bytes

    def __len__(self) -> int:
        return len(self._rows)


def _flatten(xs):
    for x in xs:
        if isinstance(x, torch.Tensor):
            yield x
        elif isinstance(x, (list, tuple)):
            yield from _flatten(x)
        elif x is not None and hasattr(x, "__dict__"):
            yield from _flatten(list(vars(x).values()))
