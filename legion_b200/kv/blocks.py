"""KV block bookkeeping: a ref-counted pool of fixed-size blocks and per-sequence block tables.

Pure host logic (no tensors): the device side is ``models.decoder.KvCache`` indexed by block id.
Behaviour follows ``src/kv/blocks.rs:1-140`` of the reference: LIFO free list (recently freed blocks
are reused first, while they may still be warm in L2), reference counts so the radix prefix cache and
several sequences can share a block, fast (device) blocks before slow (host tier) ones.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple


class OutOfBlocks(Exception):
    pass


class PyBlockPool:
    """Pure-Python pool: the fallback when the native host runtime is not built, and its executable specification."""

    def __init__(self, n_blocks: int, block_size: int, n_slow: int = 0):
        self.block_size = block_size
        self.n_blocks = n_blocks           # fast blocks: ids [0, n_blocks)
        self.n_slow = n_slow               # slow tier: ids [n_blocks, n_blocks + n_slow)
        self._ref = [0] * (n_blocks + n_slow)
        self._free_fast = list(range(n_blocks - 1, -1, -1))
        self._free_slow = list(range(n_blocks + n_slow - 1, n_blocks - 1, -1))

    # ---- queries
    @property
    def free(self) -> int:
        return len(self._free_fast) + len(self._free_slow)

    @property
    def free_fast(self) -> int:
        return len(self._free_fast)

    @property
    def used(self) -> int:
        return self.n_blocks + self.n_slow - self.free

    @property
    def total(self) -> int:
        return self.n_blocks + self.n_slow

    def refcount(self, b: int) -> int:
        return self._ref[b]

    def is_slow(self, b: int) -> bool:
        return b >= self.n_blocks

    def blocks_for(self, n_tokens: int) -> int:
        return (n_tokens + self.block_size - 1) // self.block_size

    # ---- alloc / free
    def alloc(self, n: int = 1, allow_slow: bool = True) -> List[int]:
        avail = len(self._free_fast) + (len(self._free_slow) if allow_slow else 0)
        if n > avail:
            raise OutOfBlocks(f"need {n} blocks, {avail} free")
        out = []
        for _ in range(n):
            b = self._free_fast.pop() if self._free_fast else self._free_slow.pop()
            assert self._ref[b] == 0
            self._ref[b] = 1
            out.append(b)
        return out

    def incref(self, b: int):
        assert self._ref[b] > 0, "incref of a free block"
        self._ref[b] += 1

    def decref(self, b: int):
        assert self._ref[b] > 0, "decref of a free block"
        self._ref[b] -= 1
        if self._ref[b] == 0:
            (self._free_slow if self.is_slow(b) else self._free_fast).append(b)

    def release(self, blocks: List[int]):
        for b in reversed(blocks):
            self.decref(b)


def _native():
    """The native host runtime (``legion_b200/_host.so``, built by ``build_ext.build_host``) unless
    ``LB_NATIVE_HOST=0``; None when it is not built."""
    import os
    if os.environ.get("LB_NATIVE_HOST", "1") == "0":
        return None
    try:
        from .. import _host
    except ImportError:
        return None
    _host.set_out_of_blocks(OutOfBlocks)
    return _host


NATIVE = _native()
BlockPool = NATIVE.BlockPool if NATIVE is not None else PyBlockPool


@dataclass
class CopyOp:
    src: int
    dst: int


@dataclass
class BlockTable:
    """Blocks of one sequence in position order; ``n_tokens`` cached tokens live in them."""
    blocks: List[int] = field(default_factory=list)
    n_tokens: int = 0
    n_shared: int = 0   # leading blocks borrowed from the prefix cache (never written)

    @classmethod
    def from_shared(cls, pool: BlockPool, shared: List[int], n_tokens: int) -> "BlockTable":
        for b in shared:
            pool.incref(b)
        return cls(blocks=list(shared), n_tokens=n_tokens, n_shared=len(shared))

    def capacity(self, pool: BlockPool) -> int:
        return len(self.blocks) * pool.block_size

    def ensure(self, pool: BlockPool, n_tokens: int) -> List[int]:
        """Grows the table to hold n_tokens; returns the newly allocated blocks."""
        need = pool.blocks_for(n_tokens) - len(self.blocks)
        if need <= 0:
            return []
        new = pool.alloc(need)
        self.blocks.extend(new)
        return new

    def slot(self, pool: BlockPool, pos: int) -> int:
        return self.blocks[pos // pool.block_size] * pool.block_size + pos % pool.block_size

    def slots(self, pool: BlockPool, start: int, n: int) -> List[int]:
        bs = pool.block_size
        if NATIVE is not None and n > 16:
            return NATIVE.table_slots(self.blocks, bs, start, n).tolist()
        return [self.blocks[p // bs] * bs + p % bs for p in range(start, start + n)]

    def truncate(self, pool: BlockPool, n_tokens: int):
        """Rolls the sequence back to n_tokens (speculative rejects): whole unused blocks are freed."""
        keep = pool.blocks_for(n_tokens)
        keep = max(keep, min(self.n_shared, len(self.blocks)))
        for b in reversed(self.blocks[keep:]):
            pool.decref(b)
        del self.blocks[keep:]
        self.n_tokens = min(self.n_tokens, n_tokens)

    def make_writable(self, pool: BlockPool, block_index: int) -> Optional[CopyOp]:
        """Copy-on-write of a shared block before appending into it."""
        b = self.blocks[block_index]
        if pool.refcount(b) == 1:
            return None
        nb = pool.alloc(1)[0]
        pool.decref(b)
        self.blocks[block_index] = nb
        if block_index < self.n_shared:
            self.n_shared = block_index
        return CopyOp(b, nb)

    def free(self, pool: BlockPool):
        pool.release(self.blocks)
        self.blocks = []
        self.n_tokens = 0
        self.n_shared = 0
