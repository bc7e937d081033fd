"""Block pool, block tables, radix prefix cache and recurrent-state snapshots (host bookkeeping only)."""
import random

import pytest

from legion_b200.kv import blocks as kv_blocks
from legion_b200.kv.blocks import BlockTable, OutOfBlocks, PyBlockPool
from legion_b200.kv.radix import RadixCache
from legion_b200.kv.saved_states import SavedStates, prefix_hash_at, prefix_hashes

IMPLS = ["python"] + (["native"] if kv_blocks.NATIVE is not None else [])


@pytest.fixture(params=IMPLS)
def BlockPool(request):
    """Both implementations of the pool (and, through it, of the radix tree) run the same assertions."""
    return PyBlockPool if request.param == "python" else kv_blocks.NATIVE.BlockPool


def test_native_host_runtime_is_the_default():
    """With the extension built, the engine's pool and prefix cache are the C++ ones."""
    if kv_blocks.NATIVE is None:
        pytest.skip("native host runtime not built")
    assert kv_blocks.BlockPool is kv_blocks.NATIVE.BlockPool
    p = kv_blocks.BlockPool(4, 4)
    assert type(RadixCache(p)).__module__.endswith("_host")
    t = BlockTable()
    t.ensure(p, 16)
    assert t.slots(p, 0, 16) == [t.blocks[i // 4] * 4 + i % 4 for i in range(16)]


def test_native_pack_decode_record():
    """The packed decode record: int64 KV cells, tokens, positions, cu_q, context lengths, state slots, block table;
    padding rows write no cell, read context length 1 and use the spare state slot."""
    if kv_blocks.NATIVE is None:
        pytest.skip("native host runtime not built")
    import torch
    B, W, bs = 4, 5, 4
    buf = torch.full((2 * B + B + B + B + 1 + B + B + B * W,), 77, dtype=torch.int32)
    kv_blocks.NATIVE.pack_decode(buf.numpy(), B, W, bs, 9, [7, 8], [5, 2], [0, 1], [[3, 4], [6]])
    assert buf[:2 * B].view(torch.int64).tolist() == [4 * 4 + 1, 6 * 4 + 2, -1, -1]
    rest = buf[2 * B:].tolist()
    assert rest[:4] == [7, 8, 0, 0] and rest[4:8] == [5, 2, 0, 0] and rest[8:13] == [0, 1, 2, 3, 4]
    assert rest[13:17] == [6, 3, 1, 1] and rest[17:21] == [0, 1, 9, 9]
    assert rest[21:] == [3, 4, 0, 0, 0, 6, 0, 0, 0, 0] + [0] * 10
    with pytest.raises(IndexError):
        kv_blocks.NATIVE.pack_decode(buf.numpy(), B, W, bs, 9, [7], [40], [0], [[3, 4]])


def test_pool_refcounts_and_lifo(BlockPool):
    p = BlockPool(4, 16, n_slow=2)
    a = p.alloc(3)
    assert a == [0, 1, 2] and p.free == 3 and p.free_fast == 1
    p.incref(1)
    p.release(a)
    assert p.refcount(1) == 1 and p.free == 5
    assert p.alloc(1) == [0]            # most recently freed fast block first
    b = p.alloc(2)
    assert b == [2, 3]
    assert p.is_slow(p.alloc(1)[0])     # fast blocks exhausted -> slow tier
    with pytest.raises(OutOfBlocks):
        p.alloc(5)
    with pytest.raises(AssertionError):
        p.decref(5)


def test_block_table_grow_truncate_cow(BlockPool):
    p = BlockPool(8, 4)
    t = BlockTable()
    t.ensure(p, 10)
    assert len(t.blocks) == 3 and t.slot(p, 5) == t.blocks[1] * 4 + 1
    t.truncate(p, 4)
    assert len(t.blocks) == 1 and p.free == 7
    shared = BlockTable.from_shared(p, t.blocks, 4)
    assert p.refcount(t.blocks[0]) == 2
    op = shared.make_writable(p, 0)
    assert op is not None and op.src == t.blocks[0] and shared.blocks[0] != t.blocks[0]
    assert p.refcount(t.blocks[0]) == 1
    shared.free(p)
    t.free(p)
    assert p.free == 8


def test_radix_match_insert_split_evict(BlockPool):
    p = BlockPool(32, 4)
    r = RadixCache(p)
    toks = list(range(20))
    blocks = p.alloc(5)
    assert r.insert(toks, blocks) == 5
    p.release(blocks)                              # the cache keeps its own references
    assert p.free == 27
    b, n, h = r.match_prefix(toks[:11])
    assert n == 8 and b == blocks[:2]
    r.unlock(h)
    # diverging continuation splits the edge after 2 blocks
    other = toks[:8] + [99, 98, 97, 96, 95]
    nb = p.alloc(1)
    assert r.insert(other, blocks[:2] + nb) == 1
    p.release(nb)
    b2, n2, h2 = r.match_prefix(other)
    assert n2 == 12 and b2 == blocks[:2] + nb
    # the locked path survives eviction, the other branch goes
    freed = r.evict(100)
    assert freed == 3 and r.n_cached_blocks == 3
    r.unlock(h2)
    assert r.evict(100) == 3 and p.free == 32
    assert r.match_prefix(toks)[1] == 0


def test_radix_random_against_dict_model(BlockPool):
    rng = random.Random(0)
    p = BlockPool(4096, 2)
    r = RadixCache(p)
    seqs = []
    for _ in range(60):
        base = rng.choice(seqs)[:rng.randrange(0, 12) * 2] if seqs and rng.random() < 0.7 else []
        s = base + [rng.randrange(4) for _ in range(rng.randrange(2, 16))]
        blocks, matched, h = r.match_prefix(s, lock=False)
        want = 0
        for other in seqs:
            k = 0
            while k + 2 <= min(len(s), len(other) // 2 * 2) and s[k:k + 2] == other[k:k + 2]:
                k += 2
            want = max(want, k)
        assert matched == want
        new = p.alloc(len(s) // 2 - len(blocks))
        r.insert(s, blocks + new)
        p.release(new)
        seqs.append(s)


def test_saved_states_anchor_tail_lru():
    s = SavedStates(range(10, 13), block=4)
    toks = list(range(30))
    assert s.save_points(30, 0) == [28] and s.save_points(30, 0, interval=8) == [8, 16, 24, 28]
    assert s.save_points(30, 28) == []
    slot, ev = s.reserve()
    s.store(toks, 8, slot)
    slot2, _ = s.reserve()
    s.store(toks, 22, slot2, kind="tail", tail_block=7)
    assert s.find(toks, 29).n_tokens == 22 and s.find(toks, 21).n_tokens == 8
    assert s.find(toks[:7] + [0] * 20, 26) is None
    assert s.find(toks[:20] + [0, 0, 0], 22).n_tokens == 8
    slot3, _ = s.reserve()
    s.store(toks, 16, slot3)
    s.find(toks, 9)                                # touch the 8-token anchor
    slot4, evicted = s.reserve()                    # LRU is now the tail save
    assert evicted is not None and evicted.tail_block == 7 and slot4 == slot2
    assert prefix_hashes(toks, 4)[1] == prefix_hashes(toks[:8], 4)[1]
    assert prefix_hash_at(toks, 10, 4) != prefix_hash_at(toks, 11, 4)
