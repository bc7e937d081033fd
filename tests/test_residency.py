"""Expert cache (offload) logic on the CPU backing: remap, LRU-by-heat victims, counters, and engine output
identical to the all-resident run."""
import pytest
import torch

from legion_b200.config import tiny_gqa_moe
from legion_b200.engine.lm import EngineConfig, build_engine
from legion_b200.models.weights import random_weights
from legion_b200.residency.experts import ExpertCache, slots_for_budget


def test_cache_remap_and_eviction():
    E, F, H = 6, 4, 8
    gu = torch.arange(E, dtype=torch.float32)[:, None, None].expand(E, 2 * F, H).contiguous()
    dn = torch.arange(E, dtype=torch.float32)[:, None, None].expand(E, H, F).contiguous()
    c = ExpertCache(gu, dn, n_slots=3, device="cpu")
    ids = torch.tensor([[0, 4], [4, 5]], dtype=torch.int32)
    slots = c.prepare(ids)
    g, d = c.weights()
    for t in range(2):
        for j in range(2):
            assert float(g[slots[t, j]][0, 0]) == float(ids[t, j])     # the slot holds that expert's weights
    assert c.stats.misses == 2 and c.stats.hits == 1                    # 0 was seeded, 4 and 5 were not
    c.prepare(torch.tensor([[4, 5]], dtype=torch.int32))
    assert c.stats.hits == 3
    # expert 0 is now the coldest resident one: a new expert replaces it, not 4 or 5
    c.prepare(torch.tensor([[3, 4]], dtype=torch.int32))
    assert c.slot_of[0] == -1 and c.slot_of[4] >= 0 and c.slot_of[5] >= 0 and c.slot_of[3] >= 0
    with pytest.raises(RuntimeError):
        c.prepare(torch.tensor([[0, 1, 2, 3]], dtype=torch.int32))
    assert c.stats.bytes_copied == c.bytes_per_expert * c.stats.misses
    assert slots_for_budget(tiny_gqa_moe(), 1.0) >= 2


def test_engine_with_offloaded_experts_matches_resident():
    cfg = tiny_gqa_moe()
    w = random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05)
    prompt = torch.randint(0, 255, (60,), generator=torch.Generator().manual_seed(1)).tolist()
    ec = dict(ctx_size=256, max_seqs=2, block_size=16, prefill_chunk=16, max_batch_tokens=16, prefix_cache=False)
    a = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(**ec))
    want = a.generate_text(tokens=prompt, max_tokens=10, ignore_eos=True).token_ids
    a.shutdown()
    b = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(**ec), start=False)
    b.model.offload_experts(n_slots=8)
    b.start()
    got = b.generate_text(tokens=prompt, max_tokens=10, ignore_eos=True).token_ids
    stats = [c.stats for c in b.model.expert_cache.values()]
    b.shutdown()
    assert got == want
    assert all(s.steps > 0 for s in stats)


def test_engine_with_ssd_expert_tier_matches_resident(tmp_path):
    """Experts in one file per layer, a small RAM tier, fewer HBM slots than experts: same tokens as all-resident."""
    cfg = tiny_gqa_moe()
    w = random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05)
    prompt = torch.randint(0, 255, (60,), generator=torch.Generator().manual_seed(1)).tolist()
    ec = dict(ctx_size=256, max_seqs=2, block_size=16, prefill_chunk=2, max_batch_tokens=2, prefix_cache=False)
    a = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(**ec))
    want = a.generate_text(tokens=prompt, max_tokens=10, ignore_eos=True).token_ids
    a.shutdown()
    b = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(**ec), start=False)
    b.model.offload_experts(n_slots=5, ssd_dir=str(tmp_path / "experts"), ram_experts=3)
    b.start()
    got = b.generate_text(tokens=prompt, max_tokens=10, ignore_eos=True).token_ids
    caches = list(b.model.expert_cache.values())
    b.shutdown()
    assert got == want
    assert all(c.ssd is not None and c.host_gu is None for c in caches)
    assert sum(c.stats.ssd_reads for c in caches) > 0 and sum(c.stats.ram_hits for c in caches) > 0
    assert all(len(c.ram) <= 3 for c in caches)
    assert len(list((tmp_path / "experts").iterdir())) == len(caches)
