"""Radix prefix cache over KV blocks.

A compressed radix tree whose edges are whole blocks of ``block_size`` token ids
(``src/kv/radix.rs:38-134`` in the reference). ``match_prefix`` returns the longest cached run of full
blocks for a prompt and locks the path against eviction; ``insert`` adopts a finished prompt's blocks
(taking a reference on each newly cached block); ``evict`` frees least-recently-used unlocked leaves.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

from .blocks import NATIVE, BlockPool, PyBlockPool


class _Node:
    __slots__ = ("key", "blocks", "children", "parent", "locks", "tick")

    def __init__(self, key: Tuple[int, ...], blocks: List[int], parent: Optional["_Node"]):
        self.key = key            # token ids of this edge (len = len(blocks) * block_size)
        self.blocks = blocks
        self.children: Dict[Tuple[int, ...], _Node] = {}   # keyed by the first block's tokens
        self.parent = parent
        self.locks = 0
        self.tick = 0


class PyRadixCache:
    """Pure-Python tree: the fallback when the native host runtime is not built, and its executable specification."""

    def __init__(self, pool: BlockPool):
        self.pool = pool
        self.bs = pool.block_size
        self.root = _Node((), [], None)
        self._tick = 0
        self.n_cached_blocks = 0
        self.hit_tokens = 0
        self.lookup_tokens = 0

    def _touch(self, node: _Node):
        self._tick += 1
        node.tick = self._tick

    def _first(self, tokens: Sequence[int], off: int) -> Tuple[int, ...]:
        return tuple(tokens[off:off + self.bs])

    def _split(self, node: _Node, n_blocks: int) -> _Node:
        """Splits node's edge after n_blocks blocks; returns the new upper node."""
        cut = n_blocks * self.bs
        upper = _Node(node.key[:cut], node.blocks[:n_blocks], node.parent)
        upper.locks = node.locks
        upper.tick = node.tick
        node.parent.children[self._first(node.key, 0)] = upper
        node.key = node.key[cut:]
        node.blocks = node.blocks[n_blocks:]
        node.parent = upper
        upper.children[self._first(node.key, 0)] = node
        return upper

    def match_prefix(self, tokens: Sequence[int], lock: bool = True, max_tokens: Optional[int] = None):
        """Returns (blocks, n_tokens, handle). The handle must be given back to ``unlock``."""
        limit = len(tokens) if max_tokens is None else min(len(tokens), max_tokens)
        node = self.root
        off = 0
        blocks: List[int] = []
        while off + self.bs <= limit:
            child = node.children.get(self._first(tokens, off))
            if child is None:
                break
            n_edge = len(child.blocks)
            m = 0
            while m < n_edge and off + (m + 1) * self.bs <= limit and \
                    tuple(tokens[off + m * self.bs: off + (m + 1) * self.bs]) == child.key[m * self.bs:(m + 1) * self.bs]:
                m += 1
            if m == 0:
                break
            if m < n_edge:
                child = self._split(child, m)
            blocks.extend(child.blocks)
            off += m * self.bs
            node = child
            self._touch(node)
            if m < n_edge:
                break
        self.lookup_tokens += len(tokens)
        self.hit_tokens += off
        if lock:
            n = node
            while n is not None:
                n.locks += 1
                n = n.parent
        return blocks, off, (node if lock else None)

    def unlock(self, handle: Optional[_Node]):
        n = handle
        while n is not None:
            n.locks -= 1
            assert n.locks >= 0
            n = n.parent

    def insert(self, tokens: Sequence[int], blocks: Sequence[int]) -> int:
        """Caches the full blocks of ``tokens`` (blocks[i] holds tokens[i*bs:(i+1)*bs]). Returns how many
        blocks were newly adopted (each gets one extra reference owned by the cache)."""
        n_full = min(len(tokens) // self.bs, len(blocks))
        node = self.root
        off = 0
        i = 0
        adopted = 0
        while i < n_full:
            first = self._first(tokens, off)
            child = node.children.get(first)
            if child is None:
                key = tuple(tokens[off:n_full * self.bs])
                new = _Node(key, list(blocks[i:n_full]), node)
                for b in new.blocks:
                    self.pool.incref(b)
                adopted += len(new.blocks)
                self.n_cached_blocks += len(new.blocks)
                node.children[first] = new
                self._touch(new)
                return adopted
            n_edge = len(child.blocks)
            m = 0
            while m < n_edge and i + m < n_full and \
                    tuple(tokens[off + m * self.bs: off + (m + 1) * self.bs]) == child.key[m * self.bs:(m + 1) * self.bs]:
                m += 1
            if m < n_edge:
                child = self._split(child, m)
            self._touch(child)
            node = child
            off += m * self.bs
            i += m
        return adopted

    def _leaves(self):
        out = []
        stack = [self.root]
        while stack:
            n = stack.pop()
            if n is not self.root and not n.children:
                out.append(n)
            stack.extend(n.children.values())
        return out

    def _path_tokens(self, node: _Node) -> List[int]:
        parts = []
        n = node
        while n is not None and n is not self.root:
            parts.append(n.key)
            n = n.parent
        out: List[int] = []
        for k in reversed(parts):
            out.extend(k)
        return out

    def evict(self, n_blocks: int, on_evict=None) -> int:
        """Frees up to n_blocks cached blocks, least recently used unlocked leaves first. A leaf is
        trimmed from its tail, so a partially evicted edge keeps its prefix. ``on_evict(prefix_tokens, block)``
        is called for every block before it is released, with the tokens of the whole prefix the block ends
        (a lower tier can keep the block's contents under that key)."""
        freed = 0
        while freed < n_blocks:
            leaves = [l for l in self._leaves() if l.locks == 0]
            if not leaves:
                break
            leaf = min(leaves, key=lambda l: l.tick)
            path = self._path_tokens(leaf) if on_evict is not None else None
            while leaf.blocks and freed < n_blocks:
                b = leaf.blocks.pop()
                if on_evict is not None:
                    on_evict(path, b)
                    path = path[:len(path) - self.bs]
                leaf.key = leaf.key[:len(leaf.blocks) * self.bs]
                self.pool.decref(b)
                self.n_cached_blocks -= 1
                freed += 1
            if not leaf.blocks:
                parent = leaf.parent
                for k, v in list(parent.children.items()):
                    if v is leaf:
                        del parent.children[k]
        return freed

    def clear(self):
        self.evict(self.n_cached_blocks + 1)


def RadixCache(pool):
    """The native tree over a native pool, the Python tree over a Python pool."""
    if NATIVE is not None and isinstance(pool, NATIVE.BlockPool):
        return NATIVE.RadixCache(pool)
    return PyRadixCache(pool)
