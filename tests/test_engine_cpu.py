"""Scheduler invariants on the CPU engine (fp32 reference ops, tiny random models): whatever the batching,
chunking, caching, speculation or preemption, greedy output equals a plain single-request run token for token.
Mirrors the reference's integration tests (tests/qwen35_engine.rs, spec_engine.rs, kv_on_demand.rs)."""
import threading

import pytest
import torch

from legion_b200.config import tiny_dense, tiny_gqa_moe, tiny_hybrid_moe, tiny_mla_moe
from legion_b200.engine.lm import EngineConfig, build_engine
from legion_b200.engine.types import FinishReason, GenerateRequest, SamplingParams
from legion_b200.models.weights import random_weights

CFGS = {"hybrid": tiny_hybrid_moe, "gqa_moe": tiny_gqa_moe, "dense": tiny_dense, "mla": tiny_mla_moe}


def prompt(n, seed=1, vocab=255):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def engine(name, weights=None, **kw):
    cfg = CFGS[name]()
    base = dict(ctx_size=512, max_seqs=4, block_size=16, prefill_chunk=64, max_batch_tokens=128)
    base.update(kw)
    if weights is None:
        weights = random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05)
    return build_engine(cfg, weights=weights, engine_cfg=EngineConfig(**base))


def run(eng, toks, n=24, **sp):
    return eng.generate_text(tokens=toks, max_tokens=n, ignore_eos=True, **sp)


@pytest.fixture(scope="module")
def golden():
    out = {}
    for name in CFGS:
        eng = engine(name, prefix_cache=False)
        out[name] = [run(eng, prompt(100, s)).token_ids for s in (1, 2, 3)]
        eng.shutdown()
    return out


@pytest.mark.parametrize("name", list(CFGS))
def test_batched_equals_single(name, golden):
    eng = engine(name, prefix_cache=False)
    streams = [eng.generate(GenerateRequest(prompt_tokens=prompt(100, s), sampling=SamplingParams(max_tokens=24, ignore_eos=True)))
               for s in (1, 2, 3)]
    got = [s.collect().token_ids for s in streams]
    eng.shutdown()
    assert got == golden[name]


@pytest.mark.parametrize("name", ["hybrid", "gqa_moe"])
@pytest.mark.parametrize("chunk", [16, 100, 512])
def test_chunked_prefill_equals_one_pass(name, chunk, golden):
    eng = engine(name, prefix_cache=False, prefill_chunk=chunk, max_batch_tokens=max(chunk, 16))
    got = run(eng, prompt(100, 1)).token_ids
    eng.shutdown()
    assert got == golden[name][0]


@pytest.mark.parametrize("name", list(CFGS))
def test_prefix_cache_hit_equals_cold(name, golden):
    eng = engine(name)
    a = run(eng, prompt(100, 1))
    b = run(eng, prompt(100, 1))
    # a longer prompt sharing the first 64 tokens
    p2 = prompt(100, 1)[:64] + prompt(40, 9)
    cold = engine(name, prefix_cache=False)
    want2 = run(cold, p2).token_ids
    cold.shutdown()
    c = run(eng, p2)
    st = eng.stats()
    eng.shutdown()
    assert a.token_ids == golden[name][0] and b.token_ids == golden[name][0]
    assert a.usage.cached_tokens == 0 and b.usage.cached_tokens >= 96
    assert c.token_ids == want2
    assert c.usage.cached_tokens >= (48 if name != "hybrid" else 0)
    assert st.prefix_cache_hit_tokens > 0


def test_multi_turn_resumes_from_end_of_reply_state():
    """Hybrid model: the second turn extends prompt + reply of the first; the end-of-reply snapshot (recurrent
    state + partly filled tail block) lets it resume mid-block."""
    eng = engine("hybrid")
    p1 = prompt(70, 4)
    a = run(eng, p1, n=13)
    turn2 = p1 + a.token_ids[:-1] + prompt(20, 5)
    b = run(eng, turn2, n=8)
    cold = engine("hybrid", prefix_cache=False)
    want = run(cold, turn2, n=8).token_ids
    cold.shutdown()
    eng.shutdown()
    assert b.token_ids == want
    assert b.usage.cached_tokens == 70 + 12      # everything the first turn computed


@pytest.mark.parametrize("name,spec", [("gqa_moe", "ngram"), ("hybrid", "ngram"), ("gqa_moe", "suffix"), ("gqa_moe", "draft"),
                                       ("hybrid", "draft"), ("mla", "mtp"), ("mla", "mtp_ngram"), ("gqa_moe", "eagle3"),
                                       ("dense", "dflash")])
def test_speculative_equals_plain_greedy(name, spec, golden):
    eng = engine(name, prefix_cache=False, spec=spec, spec_k=3)
    # a repetitive prompt so that n-gram drafters actually propose
    rep = (prompt(20, 1) * 5)
    plain = engine(name, prefix_cache=False)
    want = [run(plain, prompt(100, 1)).token_ids, run(plain, rep).token_ids]
    plain.shutdown()
    got = [run(eng, prompt(100, 1)).token_ids, run(eng, rep).token_ids]
    st = eng.stats()
    eng.shutdown()
    assert got == want
    if spec == "draft":          # the draft model is the target itself: every draft is accepted
        assert st.spec_draft_tokens > 0
        if name == "gqa_moe":
            assert st.spec_accepted_tokens == st.spec_draft_tokens
        else:   # recurrent layers: one-token draft steps and multi-token verify steps round differently
            assert st.spec_accepted_tokens >= 0.85 * st.spec_draft_tokens
    if spec in ("mtp", "mtp_ngram", "eagle3", "dflash", "draft"):
        assert st.spec_verify_steps > 0
    if spec == "mtp_ngram":      # the repetitive prompt is served by look-ups, the random one by the head
        assert eng.drafter.stats["ngram_hits"] > 0 and eng.drafter.stats["mtp_chains"] > 0


def test_on_demand_admission_preempts_and_recomputes(golden):
    # 3 prompts of 100 tokens + 24 outputs need 24 blocks of 16; two fit at admission (7 blocks each) but not when they grow to 8: one is preempted
    eng = engine("gqa_moe", prefix_cache=False, kv_admission="on-demand", kv_cache_tokens=15 * 16)
    streams = [eng.generate(GenerateRequest(prompt_tokens=prompt(100, s), sampling=SamplingParams(max_tokens=24, ignore_eos=True)))
               for s in (1, 2, 3)]
    got = [s.collect().token_ids for s in streams]
    st = eng.stats()
    eng.shutdown()
    assert got == golden["gqa_moe"]
    assert st.kv_preemptions >= 1


@pytest.mark.parametrize("name", ["gqa_moe", "hybrid"])
def test_preempted_sequences_swap_to_host_and_back(golden, name):
    """With a host tier the preempted sequence's KV blocks (and recurrent state) are parked and copied back:
    same tokens as an undisturbed run, and nothing is recomputed."""
    eng = engine(name, prefix_cache=False, kv_admission="on-demand", kv_cache_tokens=15 * 16, kv_swap_gib=1.0)
    streams = [eng.generate(GenerateRequest(prompt_tokens=prompt(100, s), sampling=SamplingParams(max_tokens=24, ignore_eos=True)))
               for s in (1, 2, 3)]
    got = [s.collect().token_ids for s in streams]
    st = eng.stats()
    eng.shutdown()
    assert got == golden[name]
    assert st.kv_preemptions >= 1 and st.kv_swap_out >= 1 and st.kv_swap_in == st.kv_swap_out
    assert eng._swap_bytes == 0


def test_reserve_admission_queues_until_space(golden):
    eng = engine("gqa_moe", prefix_cache=False, kv_cache_tokens=10 * 16)    # one request at a time fits
    streams = [eng.generate(GenerateRequest(prompt_tokens=prompt(100, s), sampling=SamplingParams(max_tokens=24, ignore_eos=True)))
               for s in (1, 2)]
    got = [s.collect().token_ids for s in streams]
    eng.shutdown()
    assert got == golden["gqa_moe"][:2]


def test_oversize_request_is_refused():
    eng = engine("dense", kv_cache_tokens=64)
    with pytest.raises(ValueError):
        eng.generate(GenerateRequest(prompt_tokens=prompt(100), sampling=SamplingParams(max_tokens=200)))
    eng.shutdown()


def test_stop_string_max_tokens_and_cancel():
    eng = engine("dense")
    full = run(eng, prompt(30, 2), n=16)
    assert full.finish_reason == FinishReason.LENGTH and len(full.token_ids) == 16
    text = full.text
    if len(text) > 6:
        stop = text[3:6]
        cut = eng.generate_text(tokens=prompt(30, 2), max_tokens=16, ignore_eos=True, stop=[stop])
        assert cut.finish_reason == FinishReason.STOP_SEQUENCE
        assert cut.text == text[:text.index(stop)]
    s = eng.generate(GenerateRequest(prompt_tokens=prompt(30, 2), sampling=SamplingParams(max_tokens=400, ignore_eos=True)))
    n = 0
    for ev in s:
        if ev.kind == "text":
            n += 1
            if n == 3:
                s.cancel()
        if ev.kind == "finished":
            assert ev.finish_reason == FinishReason.CANCELLED
    assert n < 400
    eng.shutdown()


def test_sampling_is_seeded_and_respects_top_k():
    eng = engine("dense")
    a = eng.generate_text(tokens=prompt(20), max_tokens=12, ignore_eos=True, temperature=1.0, seed=7)
    b = eng.generate_text(tokens=prompt(20), max_tokens=12, ignore_eos=True, temperature=1.0, seed=7)
    c = eng.generate_text(tokens=prompt(20), max_tokens=12, ignore_eos=True, temperature=1.0, seed=8)
    g = eng.generate_text(tokens=prompt(20), max_tokens=12, ignore_eos=True)
    k1 = eng.generate_text(tokens=prompt(20), max_tokens=12, ignore_eos=True, temperature=1.5, top_k=1, seed=3)
    lp = eng.generate_text(tokens=prompt(20), max_tokens=4, ignore_eos=True, logprobs=True, top_logprobs=3)
    eng.shutdown()
    assert a.token_ids == b.token_ids and a.token_ids != c.token_ids
    assert k1.token_ids == g.token_ids           # top_k = 1 is greedy whatever the temperature
    assert len(lp.logprobs) == 4 and all(len(x.top) == 3 and x.logprob <= 0 for x in lp.logprobs)
    assert lp.token_ids == g.token_ids[:4]


def test_priority_and_fair_share_order():
    from legion_b200.engine.queue import WaitQueue
    q = WaitQueue("priority")
    q.push("lo", 0)
    q.push("hi", 5)
    q.push("lo2", 0)
    q.requeue("pre", 0)
    assert [q.pop() for _ in range(4)] == ["hi", "pre", "lo", "lo2"]
    f = WaitQueue("fcfs", fair_share=True)
    f.charge("a", 1000)
    f.push("a1", key="a")
    f.push("b1", key="b")
    assert f.pop() == "b1"


def test_even_chunks_slo_budget_and_waves():
    """Prompt chunking rules, the step-time model behind --itl-target, deterministic admission waves and the
    cost-based draft depth."""
    from legion_b200.config import tiny_dense
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    cfg = tiny_dense()
    eng = build_engine(cfg, engine_cfg=EngineConfig(ctx_size=512, max_seqs=4, block_size=16, prefill_chunk=64,
                                                    prefix_cache=False, deterministic=True, itl_target_ms=50.0),
                       start=False)
    # even chunks: 130 tokens at cap 64 -> 3 chunks of 44/43/43 instead of 64/64/2
    assert eng._chunk_len(130, 64) == 44 and eng._chunk_len(86, 64) == 43 and eng._chunk_len(43, 64) == 43
    eng.cfg.even_chunks = False
    assert eng._chunk_len(130, 64) == 64
    eng.cfg.even_chunks = True
    # step-time model: 10 ms decode steps, 0.5 ms per prompt token -> 80 prompt tokens fit a 50 ms ITL target
    for _ in range(20):
        eng._observe_step(4, 0, 10.0)
        eng._observe_step(4, 100, 60.0)
    assert 70 <= eng.slo_budget(4, False) <= 90
    assert eng.slo_budget(0, False) == 0
    # waves: the second request is not admitted while the first one runs
    prompt = list(range(1, 40))
    s1 = eng.generate(GenerateRequest(prompt_tokens=prompt, sampling=SamplingParams(max_tokens=4, ignore_eos=True)))
    eng._drain(block=False)
    eng._admit()
    eng.step()
    s2 = eng.generate(GenerateRequest(prompt_tokens=prompt, sampling=SamplingParams(max_tokens=4, ignore_eos=True)))
    eng._drain(block=False)
    eng._admit()
    assert len(eng.running) == 1 and len(eng.waiting) == 1
    for _ in range(50):
        eng._admit()
        if not eng.running and len(eng.waiting) == 0:
            break
        eng.step()
    assert s1.collect().token_ids == s2.collect().token_ids
    # draft depth: high acceptance and few sequences -> deep drafts; low acceptance and many -> none
    eng.cfg.spec_policy, eng.cfg.spec_k = "cost", 6
    eng._stats.spec_draft_tokens, eng._stats.spec_accepted_tokens = 1000, 900
    deep = eng._spec_depth(1)
    eng._stats.spec_accepted_tokens = 100
    shallow = eng._spec_depth(8)
    assert deep >= 4 and shallow <= 1


@pytest.mark.parametrize("preset", ["tiny-muse", "tiny-gemma", "tiny-nemotron-h"])
def test_more_architectures_generate_and_reuse_prefix(preset):
    """Architectures that are configurations of the same block library (NoPE / sliding-window attention, GELU and
    squared-ReLU FFNs, Mamba-2, logit scale / soft cap, (w - 1) norms, tied embeddings): chunked prefill equals one
    shot prefill, and a re-sent prompt decodes the same tokens."""
    from legion_b200.config import PRESETS
    from legion_b200.engine.lm import EngineConfig, build_engine
    cfg = PRESETS[preset]()
    prompt = torch.randint(0, 255, (100,), generator=torch.Generator().manual_seed(4)).tolist()
    outs = []
    for chunk in (128, 32):
        eng = build_engine(cfg, engine_cfg=EngineConfig(ctx_size=256, max_seqs=2, block_size=16, prefill_chunk=chunk),
                           seed=1)
        a = eng.generate_text(tokens=prompt, max_tokens=8, ignore_eos=True).token_ids
        b = eng.generate_text(tokens=prompt, max_tokens=8, ignore_eos=True).token_ids
        eng.shutdown()
        assert a == b and len(a) == 8
        outs.append(a)
    assert outs[0] == outs[1]


def test_prefix_cache_host_tier_restores_evicted_blocks():
    """A small KV pool: the first prompt's cached blocks are evicted by later prompts, their contents go to the
    host tier, and the first prompt sent again gets them back (cached tokens, same output) instead of recomputing."""
    cfg = tiny_gqa_moe()
    w = random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05)
    ec = dict(ctx_size=128, max_seqs=1, block_size=16, prefill_chunk=64, kv_cache_tokens=160, prefix_cache=True)
    eng = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(prefix_host_gib=0.01, **ec))
    base = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(**ec))
    pa = torch.randint(0, 255, (100,), generator=torch.Generator().manual_seed(1)).tolist()
    others = [torch.randint(0, 255, (100,), generator=torch.Generator().manual_seed(s)).tolist() for s in (2, 3)]
    first = eng.generate_text(tokens=pa, max_tokens=6, ignore_eos=True)
    for p in others:
        eng.generate_text(tokens=p, max_tokens=6, ignore_eos=True)
        base.generate_text(tokens=p, max_tokens=6, ignore_eos=True)
    st = eng.stats()
    assert st.prefix_host_spilled > 0
    again = eng.generate_text(tokens=pa, max_tokens=6, ignore_eos=True)
    st = eng.stats()
    want = base.generate_text(tokens=pa, max_tokens=6, ignore_eos=True)       # recomputed from scratch there
    eng.shutdown()
    base.shutdown()
    assert again.token_ids == first.token_ids == want.token_ids
    assert st.prefix_host_restored > 0 and again.usage.cached_tokens >= 32
    assert want.usage.cached_tokens < again.usage.cached_tokens


def test_repeated_conversation_does_not_pin_more_blocks():
    """Hybrid model, same prompt answered again and again: every reply saves the same ragged tail. The replaced
    snapshot must give its tail block back, so the number of free KV blocks settles instead of shrinking by one
    block per repeat."""
    eng = engine("hybrid", max_seqs=1)
    p = prompt(70, 4)
    free = []
    for _ in range(5):
        run(eng, p, n=13)
        free.append(eng.pool.free)
    eng.shutdown()
    assert free[2] == free[3] == free[4], free


def test_saved_state_store_reports_the_replaced_entry():
    from legion_b200.kv.saved_states import SavedStates
    ss = SavedStates(slots=[0, 1, 2], block=16)
    toks = list(range(40))
    gone = []
    s1, _ = ss.reserve()
    ss.store(toks, 37, s1, "tail", tail_block=7, on_replace=gone.append)
    s2, _ = ss.reserve()
    ss.store(toks, 37, s2, "tail", tail_block=9, on_replace=gone.append)
    assert [g.slot for g in gone] == [s1] and len(ss) == 1
    assert ss.find(toks, 39).tail_block == 9
    assert sorted(ss._free) == sorted({0, 1, 2} - {s2})


def test_resume_snapshot_survives_making_room():
    """A KV pool so small that admitting the second turn has to drop saved snapshots: the snapshot chosen for the
    resume must not be the one that is dropped (its tail block and state slot are about to be taken over)."""
    cfg = CFGS["hybrid"]()
    w = random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05)
    ec = dict(ctx_size=160, max_seqs=1, block_size=16, prefill_chunk=64, max_batch_tokens=128, kv_cache_tokens=176)
    eng = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(**ec))
    p1 = prompt(70, 4)
    a = run(eng, p1, n=13)
    # other conversations leave their own tail saves behind and fill the pool
    for s in (11, 12):
        run(eng, prompt(20, s), n=5)
    turn2 = p1 + a.token_ids[:-1] + prompt(60, 5)
    b = run(eng, turn2, n=8)
    cold = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(prefix_cache=False, **ec))
    want = run(cold, turn2, n=8).token_ids
    cold.shutdown()
    eng.shutdown()
    assert b.token_ids == want


def test_memory_plan_sizes_the_kv_pool_and_reports_what_fits():
    """The planner behind --kv-cache-tokens auto: blocks that fit beside weights, state slots and the kept-back
    workspace; an explicit pool that is too large is reported with the largest context that would fit."""
    from legion_b200.engine import memory_plan as mp
    G = 1 << 30
    bpb = 48 * 64 * 2 * 2 * 256 * 2                     # 48 layers, 64-token blocks, K+V, 2 kv heads of 256, bf16
    ws = mp.workspace_reserve(2048, 151936, 8192, 16, 512, 10, 512)
    assert 1 * G < ws < 8 * G
    plan = mp.fit(total_bytes=180 * G, free_bytes=120 * G, weights_bytes=58 * G, bytes_per_block=bpb, block_size=64,
                  state_bytes=2 * G, workspace_bytes=ws, max_seqs=16, ctx_size=32768, asked_tokens=0, utilisation=0.92)
    assert plan.fits and plan.n_blocks == 16 * 32768 // 64          # every sequence gets its whole context
    assert any("left unused" in n for n in plan.notes)
    tight = mp.fit(180 * G, 20 * G, 150 * G, bpb, 64, 2 * G, ws, 256, 131072, asked_tokens=0, utilisation=0.92)
    assert 0 < tight.n_blocks < 256 * 131072 // 64 and tight.kv_bytes <= 20 * G - 2 * G - ws
    assert tight.max_ctx_fit == tight.n_blocks // 256 * 64 or tight.max_ctx_fit <= tight.kv_tokens
    too_big = mp.fit(180 * G, 20 * G, 150 * G, bpb, 64, 2 * G, ws, 256, 131072, asked_tokens=256 * 131072)
    assert not too_big.fits and "does not fit" in "\n".join(too_big.lines())


def test_tool_call_parsers_glm_and_gemma4_formats():
    """GLM's key / value tags and Gemma 4's own argument notation, fed in small pieces as a stream would."""
    import json

    from legion_b200.engine.text import ToolCallParser

    def run(fmt, text, piece=5):
        p = ToolCallParser(fmt)
        out, calls = "", []
        for i in range(0, len(text), piece):
            t, c = p.push(text[i:i + piece])
            out += t
            calls += c
        t, c = p.flush()
        return out + t, calls + c

    glm = ("Let me look.\n<tool_call>get_weather\n<arg_key>city</arg_key>\n<arg_value>Paris</arg_value>\n"
           "<arg_key>days</arg_key>\n<arg_value>3</arg_value>\n<arg_key>opts</arg_key><arg_value>{\"a\": [1, 2]}</arg_value>"
           "</tool_call> done")
    text, calls = run("glm", glm)
    assert text == "Let me look.\n done" and len(calls) == 1 and calls[0]["name"] == "get_weather"
    assert json.loads(calls[0]["arguments"]) == {"city": "Paris", "days": 3, "opts": {"a": [1, 2]}}
    assert run("glm", "<tool_call><bad>\n</tool_call>")[1] == []
    gem = 'ok <|tool_call>call:get_weather{city:<|"|>東京, "x"<|"|>,days:2,deep:{on:true,list:[1,2.5,null,<|"|>a<|"|>]}}<tool_call|>!'
    text, calls = run("gemma4", gem, piece=3)
    assert text == "ok !" and calls[0]["name"] == "get_weather"
    assert json.loads(calls[0]["arguments"]) == {"city": '東京, "x"', "days": 2, "deep": {"on": True, "list": [1, 2.5, None, "a"]}}
    assert run("gemma4", "<|tool_call>call:f{a:}<tool_call|>")[1] == []            # malformed: no call
    assert run("hermes", "<tool_call>{\"name\": \"f\", \"arguments\": {\"a\": 1}}</tool_call>")[1][0]["name"] == "f"


def test_sliding_window_rings_equal_full_paging():
    """Sliding-window layers on a short ring of blocks per sequence (window + one step) give the tokens of full
    paging: prompts several windows long, chunked prefill through the ring, batched decode, n-gram speculation."""
    import torch
    from legion_b200.config import PRESETS
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    from legion_b200.models.weights import random_weights
    cfg = PRESETS["tiny-gemma"]()
    w = random_weights(cfg, "cpu", torch.float32, seed=11, std=0.08)
    prompts = [list(range(7, 7 + n)) + [5, 6, 7, 5, 6, 7, 5, 6] for n in (150, 61, 97)]
    base = dict(ctx_size=512, max_seqs=4, block_size=16, prefill_chunk=32, max_batch_tokens=96, prefix_cache=False)

    def run(**kw):
        eng = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(**base, **kw))
        streams = [eng.generate(GenerateRequest(prompt_tokens=p, sampling=SamplingParams(max_tokens=40, ignore_eos=True)))
                   for p in prompts]
        outs = [s.collect().token_ids for s in streams]
        info = (eng.ring_len, eng.kv.k[0].shape[0], eng.kv.k[1].shape[0])
        eng.shutdown()
        return outs, info

    full, (l0, n_swa, n_glob) = run()
    assert l0 == 0 and n_swa == n_glob
    ring, (l1, r_swa, r_glob) = run(kv_rings=True)
    assert l1 == (48 + 32 + 15) // 16 + 1 and r_swa == l1 * (4 + 1) and r_glob == n_glob and r_swa < n_glob
    assert ring == full
    spec, _ = run(kv_rings=True, spec="ngram", spec_k=3)
    assert spec == full
    # the rings travel with the state snapshots: a repeated prompt resumes from the prefix cache (its window history
    # comes back with the snapshot) and continues with the same tokens; an extended prompt resumes at the anchor
    cached = dict(base, prefix_cache=True)
    eng = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(**cached, kv_rings=True))
    first = eng.generate_text(tokens=prompts[0], max_tokens=12, ignore_eos=True)
    again = eng.generate_text(tokens=prompts[0], max_tokens=12, ignore_eos=True)
    longer = eng.generate_text(tokens=prompts[0] + first.token_ids[:5] + [9, 9, 9], max_tokens=6, ignore_eos=True)
    eng.shutdown()
    ref_eng = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(**base))
    want_longer = ref_eng.generate_text(tokens=prompts[0] + first.token_ids[:5] + [9, 9, 9], max_tokens=6, ignore_eos=True)
    ref_eng.shutdown()
    assert first.token_ids == full[0][:12] and again.token_ids == first.token_ids
    assert again.usage.cached_tokens >= 64 and longer.usage.cached_tokens >= 64
    assert longer.token_ids == want_longer.token_ids


def test_eagle3_head_from_a_checkpoint_directory(tmp_path):
    """An EAGLE-3 checkpoint (config flags, own head shape, reduced draft vocabulary with ``d2t`` offsets, biases,
    ``layers.0`` naming) loads into the drafter: speculation with it equals plain greedy decoding, the flags change
    what the head computes, and a head that does not fit the target is refused."""
    import json
    import pytest
    import torch
    from legion_b200.config import ModelConfig
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.loaders.safetensors_io import save_file
    from legion_b200.models.weights import random_weights
    from legion_b200.spec.drafters import Eagle3Config, Eagle3Head
    cfg = ModelConfig(arch="qwen3", n_layer=4, hidden=64, vocab=512, n_head=4, n_kv_head=2, head_dim=16, dense_ff=128)
    w = random_weights(cfg, "cpu", torch.float32, seed=2, std=0.08)
    H, nq, nkv, D, F, DV = 64, 2, 1, 32, 96, 200
    g = torch.Generator().manual_seed(0)
    r = lambda *sh: torch.randn(*sh, generator=g) * 0.05       # noqa: E731
    d2t_target = torch.sort(torch.randperm(512, generator=g)[:DV]).values
    tensors = {"fc.weight": r(H, 3 * H), "lm_head.weight": r(DV, H), "norm.weight": torch.ones(H) + r(H),
               "input_norm.weight": torch.ones(3 * H) + r(3 * H), "d2t": (d2t_target - torch.arange(DV)).long(),
               "t2d": torch.zeros(512, dtype=torch.bool)}
    L = "layers.0"
    for n, sh in (("self_attn.q_proj", (nq * D, 2 * H)), ("self_attn.k_proj", (nkv * D, 2 * H)),
                  ("self_attn.v_proj", (nkv * D, 2 * H)), ("self_attn.o_proj", (H, nq * D)), ("mlp.gate_proj", (F, H)),
                  ("mlp.up_proj", (F, H)), ("mlp.down_proj", (H, F))):
        tensors[f"{L}.{n}.weight"] = r(*sh)
    for n in ("input_layernorm", "hidden_norm", "post_attention_layernorm"):
        tensors[f"{L}.{n}.weight"] = torch.ones(H) + r(H)
    for n, k in (("q_proj", nq * D), ("k_proj", nkv * D), ("v_proj", nkv * D)):
        tensors[f"{L}.self_attn.{n}.bias"] = r(k)
    d = tmp_path / "eagle3"
    d.mkdir()
    save_file(tensors, str(d / "model.safetensors"))
    conf = {"architectures": ["LlamaForCausalLMEagle3"], "hidden_size": H, "intermediate_size": F, "num_attention_heads": nq,
            "num_key_value_heads": nkv, "head_dim": D, "vocab_size": 512, "draft_vocab_size": DV, "num_hidden_layers": 1,
            "rms_norm_eps": 1e-5, "rope_theta": 50000.0, "max_position_embeddings": 2048, "attention_bias": True,
            "norm_before_fc": True, "eagle_config": {"eagle_aux_hidden_state_layer_ids": [0, 1, 3],
                                                     "norm_before_residual": True}}
    (d / "config.json").write_text(json.dumps(conf))
    hc = Eagle3Config.parse(conf)
    assert (hc.n_aux, hc.layer_ids, hc.draft_vocab, hc.attention_bias, hc.norm_before_residual, hc.norm_before_fc,
            hc.fc_norm, hc.rope_theta) == (3, [0, 1, 3], DV, True, True, True, False, 50000.0)
    head = Eagle3Head.from_checkpoint(str(d), cfg, "cpu", torch.float32)
    assert torch.equal(head.d2t, d2t_target) and head.cos_sin is not None and "b_qkv" in head.w
    feats = [torch.randn(5, H) for _ in range(3)]
    fused = head.fuse(feats)
    cat = torch.cat(feats, -1)
    want = (cat * torch.rsqrt(cat.pow(2).mean(-1, keepdim=True) + 1e-5) * tensors["input_norm.weight"]) @ tensors["fc.weight"].t()
    assert torch.allclose(fused, want, atol=1e-5)
    ec = dict(ctx_size=256, max_seqs=2, block_size=16, prefill_chunk=64, max_batch_tokens=128)
    prompt = list(range(7, 60)) + [7, 8, 9, 7, 8, 9]
    plain = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(**ec))
    want_toks = plain.generate_text(tokens=prompt, max_tokens=20, ignore_eos=True).token_ids
    plain.shutdown()
    spec = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(spec="eagle3", spec_k=3, spec_draft_model=str(d), **ec))
    assert spec.drafter.capture_layers == [0, 1, 3] and spec.drafter.k.shape[2:] == (nkv, D)
    got = spec.generate_text(tokens=prompt, max_tokens=20, ignore_eos=True)
    drafted = spec.stats().spec_draft_tokens
    spec.shutdown()
    assert got.token_ids == want_toks and drafted > 0
    conf_bad = dict(conf, hidden_size=128)
    (d / "config.json").write_text(json.dumps(conf_bad))
    with pytest.raises(ValueError):
        Eagle3Head.from_checkpoint(str(d), cfg, "cpu", torch.float32)
    with pytest.raises(ValueError):
        Eagle3Config.parse(dict(conf, num_hidden_layers=2))


def test_adaptive_draft_depth_follows_acceptance_and_costs():
    """The depth model's pieces, then the engine under ``spec_policy="adaptive"``: tokens equal plain decoding; a text
    the n-gram drafter predicts well keeps drafting deep, one it cannot predict stops drafting (but keeps probing)."""
    import torch
    from legion_b200.config import PRESETS
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.models.weights import random_weights
    from legion_b200.spec.depth import AdaptiveState, DepthModel, chain_gain
    good, bad = AdaptiveState(), AdaptiveState()
    assert abs(good.gain(3) - chain_gain(0.6, 3)) < 1e-9 and good.cap(0.5, 8) == 1
    for _ in range(25):
        good.update(4, 4, 4)
        bad.update(4, 0, 4)
    assert good.cap(0.5, 8) == 8 and bad.cap(0.5, 8) == 0 and good.gain(4) > 4.5 and bad.gain(4) < 1.1
    half = AdaptiveState()
    for _ in range(40):
        half.update(4, 2, 4)               # always two accepted, then a rejection
    assert 0.6 < half.rate < 0.72 and abs(half.gain(2) - 3.0) < 0.05 and abs(half.gain(6) - 3.0) < 0.05
    m = DepthModel(6)
    for rows, ms in ((2, 5.0), (4, 5.2), (8, 5.5), (16, 9.0), (32, 20.0)):
        m.observe_verify(rows, ms)
    assert m.choose([good, good], 2) in (3, 6) and m.choose([bad, bad], 2) == 0
    # verify rows that cost as much as whole steps make even a perfect drafter shallow
    steep = DepthModel(6)
    for rows, ms in ((2, 5.0), (4, 10.0), (8, 20.0), (16, 40.0)):
        steep.observe_verify(rows, ms)
    assert steep.choose([half, half], 2) <= 1

    cfg = PRESETS["tiny-dense"]()
    w = random_weights(cfg, "cpu", torch.float32, seed=5, std=0.08)
    ec = dict(ctx_size=512, max_seqs=2, block_size=16, prefill_chunk=128, max_batch_tokens=256)
    rep = [11, 12, 13, 14, 15, 16] * 20                   # whatever follows, the drafter proposes the repeating cycle
    plain = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(**ec))
    want = plain.generate_text(tokens=rep, max_tokens=40, ignore_eos=True).token_ids
    plain.shutdown()
    eng = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(spec="ngram", spec_k=4, spec_policy="adaptive", **ec))
    got = eng.generate_text(tokens=rep, max_tokens=40, ignore_eos=True)
    st = eng.stats()
    eng.shutdown()
    assert got.token_ids == want
    # a random model does not continue the cycle: acceptance collapses and the policy stops paying for deep drafts
    assert st.spec_draft_tokens < 4 * 40 * 0.6


def test_reply_starts_inside_reasoning_when_the_prompt_left_it_open():
    """A template that ends the prompt with the reasoning opener (thinking models): the reply's text goes to the
    reasoning channel from its first token; the same model after a prompt without the opener answers on the text
    channel; the vocabulary's further end-of-turn tokens stop a reply."""
    eng = engine("dense")
    tok = eng.tok
    assert eng.chat_format.prompt_mode == "from_prompt" and tok.token_to_id("<|im_end|>") in eng.eos_ids
    kinds = {}
    for label, text in (("open", "<|im_start|>assistant\n<think>\n"), ("closed", "<|im_start|>assistant\n")):
        st = eng.generate(GenerateRequest(prompt=text, sampling=SamplingParams(max_tokens=12, ignore_eos=True)))
        kinds[label] = {ev.kind for ev in st if ev.kind in ("text", "reasoning") and ev.text}
    eng.shutdown()
    assert kinds["open"] == {"reasoning"} and kinds["closed"] == {"text"}
