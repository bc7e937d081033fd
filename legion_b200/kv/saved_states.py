"""Recurrent-state snapshots for the prefix cache of hybrid (Gated DeltaNet / Mamba) models.

KV blocks alone cannot resume a hybrid model in the middle of a prompt: the recurrent layers need the
state as of the resume position. Snapshots are taken at block boundaries while a prompt is prefilled
(anchor = the prompt's last full block, plus optional spaced saves) and once at the end of a reply
(tail save, which also keeps the partly filled last KV block alive). A new prompt resumes at the
longest snapshot position that is covered by cached KV blocks. Mirrors the behaviour of
``src/engine/saved_states.rs:1-120,186-217`` in the reference; slots are recycled LRU.
"""
from __future__ import annotations

import hashlib
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple


def prefix_hashes(tokens: Sequence[int], block: int) -> List[bytes]:
    """hashes[i] identifies tokens[: (i + 1) * block] (chained, so computing all of them is O(n))."""
    out = []
    h = b""
    for i in range(len(tokens) // block):
        m = hashlib.blake2b(digest_size=16)
        m.update(h)
        m.update(struct.pack(f"<{block}i", *tokens[i * block:(i + 1) * block]))
        h = m.digest()
        out.append(h)
    return out


def prefix_hash_at(tokens: Sequence[int], n: int, block: int) -> bytes:
    """Identifier of tokens[:n] for any n (full-block chain plus the ragged tail)."""
    hs = prefix_hashes(tokens[:n], block)
    m = hashlib.blake2b(digest_size=16)
    m.update(hs[-1] if hs else b"")
    tail = tokens[(n // block) * block:n]
    m.update(struct.pack(f"<{len(tail)}i", *tail))
    m.update(b"tail")
    return m.digest()


@dataclass
class Saved:
    slot: int
    n_tokens: int
    key: bytes
    kind: str                 # "anchor" | "spaced" | "tail"
    tail_block: Optional[int] = None   # KV block holding the ragged tail (tail saves only)
    tick: int = 0


class SavedStates:
    def __init__(self, slots: Sequence[int], block: int):
        """``slots`` are the state-pool slot ids reserved for snapshots."""
        self.block = block
        self._free = list(slots)
        self._by_key: Dict[Tuple[int, bytes], Saved] = {}
        self._tick = 0
        self.hits = 0

    def __len__(self):
        return len(self._by_key)

    def _touch(self, s: Saved):
        self._tick += 1
        s.tick = self._tick

    def save_points(self, prompt_len: int, resumed: int, interval: int = 0) -> List[int]:
        """Positions (multiples of the block size, > resumed, < prompt_len) at which to snapshot while
        prefilling: the last full block boundary, plus every ``interval`` tokens when requested."""
        pts = set()
        last = ((prompt_len - 1) // self.block) * self.block
        if last > resumed:
            pts.add(last)
        if interval > 0:
            step = max(self.block, (interval // self.block) * self.block)
            p = ((resumed // step) + 1) * step
            while p < prompt_len:
                pts.add(p)
                p += step
        return sorted(pts)

    def find(self, tokens: Sequence[int], max_tokens: int) -> Optional[Saved]:
        """Longest snapshot of a prefix of ``tokens`` with at most max_tokens tokens."""
        best = None
        hs = prefix_hashes(tokens[:max_tokens], self.block)
        for i in range(len(hs) - 1, -1, -1):
            s = self._by_key.get(((i + 1) * self.block, hs[i]))
            if s is not None:
                best = s
                break
        # tail saves: any position, exact prefix match
        for (n, key), s in self._by_key.items():
            if s.kind == "tail" and n <= max_tokens and (best is None or n > best.n_tokens):
                if prefix_hash_at(tokens, n, self.block) == key:
                    best = s
        if best is not None:
            self._touch(best)
            self.hits += 1
        return best

    def reserve(self) -> Tuple[Optional[int], Optional[Saved]]:
        """Returns (slot, evicted): a free slot, or the LRU snapshot's slot (the caller releases the
        evicted entry's tail block)."""
        if self._free:
            return self._free.pop(), None
        if not self._by_key:
            return None, None
        victim = min(self._by_key.values(), key=lambda s: s.tick)
        del self._by_key[(victim.n_tokens, victim.key)]
        return victim.slot, victim

    def store(self, tokens: Sequence[int], n_tokens: int, slot: int, kind: str = "anchor",
              tail_block: Optional[int] = None, on_replace=None) -> Saved:
        """Records a snapshot. An entry with the same position and prefix is replaced: its slot goes back to the
        free list and ``on_replace(old)`` lets the owner of the KV pool give back the reference that the old
        entry held on its tail block (without it every repeat of the same conversation would pin one more block).
        """
        if n_tokens % self.block == 0 and kind != "tail":
            key = prefix_hashes(tokens[:n_tokens], self.block)[-1]
        else:
            kind = "tail"
            key = prefix_hash_at(tokens, n_tokens, self.block)
        old = self._by_key.get((n_tokens, key))
        if old is not None:
            self._free.append(old.slot)
            if on_replace is not None:
                on_replace(old)
            old.tail_block = None
        s = Saved(slot, n_tokens, key, kind, tail_block)
        self._by_key[(n_tokens, key)] = s
        self._touch(s)
        return s

    def drop(self, s: Saved):
        if self._by_key.pop((s.n_tokens, s.key), None) is not None:
            self._free.append(s.slot)

    def entries(self) -> List[Saved]:
        return list(self._by_key.values())
