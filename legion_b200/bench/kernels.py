"""Kernel micro-benchmarks: device-timed (CUDA events, warm-up, L2 flush between iterations), reported
as achieved TFLOP/s or GB/s and as a fraction of the measured peaks in ``MEASURED_PEAKS.json``.

Usage: ``python -m legion_b200.bench.kernels [--only gemm,moe,decode_attn,prefill_attn] [--json out.json]``
The reference ships one hidden ``legion <kernel>-bench`` command per custom kernel (``src/cli/mod.rs:109-215``);
this module is their counterpart.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None
CASE = {"tokens": None, "attn": None, "gemm": None}


def flush_l2():
    """Evicts L2 by READING a buffer twice its size: the lines it leaves behind are clean, so the timed kernel
    does not pay for write-backs of the flush itself."""
    global _flush
    if _flush is None:
        _flush = torch.zeros(64 << 20, dtype=torch.int32, device="cuda")
    _flush.sum()


ITERS = {"iters": None, "warmup": None}


def timeit(fn, iters=10, warmup=3, flush=True):
    iters = ITERS["iters"] or iters
    warmup = ITERS["warmup"] if ITERS["warmup"] is not None else warmup
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


_flush_graph_ms = {}


def timeit_graph(fn, iters=5, warmup=3, reps=20):
    """Device time of one call of ``fn`` replayed from a CUDA graph (no host launch cost in the number) with a cold
    L2. One graph holds ``reps`` x (L2 flush, fn) back to back so the GPU stays busy and at its working clocks (a
    lone kernel between two synchronisations runs at idle clocks and reads several times too slow); the time of a
    graph of ``reps`` flushes alone is subtracted."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()

    def capture(body):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                flush_l2()
                body()
        return g

    def run(g):
        ts = []
        for _ in range(ITERS["iters"] or iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g.replay()                      # brings the clocks up
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        ts.sort()
        return ts[len(ts) // 2]
    flush_l2()
    if reps not in _flush_graph_ms:
        _flush_graph_ms[reps] = run(capture(lambda: None))
    total = run(capture(fn))
    return max(0.0, total - _flush_graph_ms[reps]) / reps


def bench_layer_parts(rows):
    """The pieces of one decode step of a 30B-A3B-shaped layer (16 users, 8K context), each replayed from a CUDA
    graph: which kernel the step time goes to."""
    from legion_b200.ops import sm100
    hbm, tf, src = peaks()
    T, H, E, k, F, Hq, Hkv, D, page, ctx = 16, 2048, 128, 8, 768, 32, 4, 128, 64, 8256
    dev = "cuda"
    x = torch.randn(T, H, device=dev).bfloat16()
    res = torch.randn(T, H, device=dev).bfloat16()
    nw = torch.ones(H, device=dev)
    w_qkv = (torch.randn((Hq + 2 * Hkv) * D, H, device=dev) * 0.02).bfloat16()
    w_o = (torch.randn(H, Hq * D, device=dev) * 0.02).bfloat16()
    w_r = (torch.randn(E, H, device=dev) * 0.02).bfloat16()
    wgu = (torch.randn(E, 2 * F, H, device=dev) * 0.02).bfloat16()
    wd = (torch.randn(E, H, F, device=dev) * 0.02).bfloat16()
    attn_in = torch.randn(T, Hq * D, device=dev).bfloat16()
    nb = T * ((ctx + page - 1) // page)
    kc = torch.randn(nb, page, Hkv, D, device=dev).bfloat16()
    vc = torch.randn(nb, page, Hkv, D, device=dev).bfloat16()
    bt = torch.arange(nb, device=dev, dtype=torch.int32).view(T, -1)
    q = torch.randn(T, Hq, D, device=dev).bfloat16()
    cl = torch.full((T,), ctx, device=dev, dtype=torch.int32)
    routing = sm100.router(x, w_r, k)
    ids, wts = routing

    def add(name, fn, byts=0):
        ms = timeit_graph(fn)
        rows.append(dict(kernel="layer_part", part=name, us=ms * 1e3, gbs=byts / ms / 1e6 if byts else 0.0,
                         frac_hbm=byts / ms / 1e6 / hbm if byts else 0.0, peaks=src))
        print(rows[-1], flush=True)

    add("rmsnorm", lambda: sm100.rmsnorm(x, nw, 1e-6, residual=res))
    add("qkv_gemm", lambda: sm100.linear(x, w_qkv), w_qkv.numel() * 2)
    add("o_gemm", lambda: sm100.linear(attn_in, w_o, residual=res), w_o.numel() * 2)
    kv_bytes = T * ctx * Hkv * D * 2 * 2
    for s in (CASE["tokens"] or (4, 8, 9, 10, 12, 16, 22, 33)):
        add(f"decode_attn_splits{s}", lambda: sm100.paged_decode(q, kc, vc, bt, cl, D ** -0.5, n_splits=s,
                                                                   max_ctx=ctx), kv_bytes)
    add("router_route", lambda: sm100.router(x, w_r, k), w_r.numel() * 2)
    add("norm_router_route", lambda: sm100.router(x, w_r, k, norm=(nw, 1e-6, 0.0)), w_r.numel() * 2)
    n_act = int(torch.unique(ids).numel())
    add("moe_experts_dense", lambda: sm100.moe_experts(x, ids, wts, wgu, wd, F, residual=res, norm=(nw, 1e-6, 0.0),
                                                       routing=routing), n_act * 3 * H * F * 2)
    from legion_b200.ops.sm100 import QWeight
    qgu = QWeight(torch.randint(0, 256, (E, 2 * F, H // 2), device=dev, dtype=torch.uint8),
                  torch.randint(48, 64, (E, 2 * F, H // 16), device=dev, dtype=torch.uint8),
                  torch.ones(2 * E, device=dev))
    qd = QWeight(torch.randint(0, 256, (E, H, F // 2), device=dev, dtype=torch.uint8),
                 torch.randint(48, 64, (E, H, F // 16), device=dev, dtype=torch.uint8), torch.ones(E, device=dev))
    add("moe_experts_dense_nvfp4", lambda: sm100.moe_experts(x, ids, wts, qgu, qd, F, residual=res,
                                                            norm=(nw, 1e-6, 0.0), routing=routing),
        n_act * 3 * H * F * 9 // 16)
    add("moe_experts_gather", lambda: sm100.moe_experts(x, ids, wts, wgu, wd, F, residual=res, norm=(nw, 1e-6, 0.0)),
        n_act * 3 * H * F * 2)
    # the MoE pieces on their own
    C = sm100.ext()
    ws = sm100.Workspace.get(torch.device(dev))
    plan = sm100.MoePlan(T, k, E, 32, dev)
    P = T * k
    plan.x_sorted = torch.zeros(P + 32, H, dtype=torch.bfloat16, device=dev)
    plan.h_sorted = torch.zeros(P + 32, F, dtype=torch.bfloat16, device=dev)
    plan.y_pairs = torch.zeros(P, H, dtype=torch.bfloat16, device=dev)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    normed = torch.empty_like(out)
    f_plan = lambda: C.moe_plan_gather(ids, wts, 0, E, 32, plan.counts, plan.offsets, plan.sorted_token,
                                       plan.sorted_pair, plan.sorted_w, plan.tile_group, plan.tile_tok0,
                                       plan.tile_ntok, plan.meta, x, plan.x_sorted)
    f_gu = lambda: C.wgemm(wgu.view(E * 2 * F, H), plan.x_sorted, plan.h_sorted, None, None, None, F, True, F, 32, 1,
                           None, None, ws.status, plan.tile_group, plan.tile_tok0, plan.tile_ntok, plan.meta,
                           plan.max_tiles, 2 * F, 0, [])
    f_dn = lambda: C.wgemm(wd.view(E * H, F), plan.h_sorted, plan.y_pairs, None, plan.sorted_w, plan.sorted_pair, H,
                           False, 0, 32, 1, None, None, ws.status, plan.tile_group, plan.tile_tok0, plan.tile_ntok,
                           plan.meta, plan.max_tiles, H, 0, [])
    f_cb = lambda: C.moe_combine(plan.y_pairs, ids, 0, E, None, None, res, out, nw, 1e-6, 0.0, normed)
    f_plan()
    add("moe.plan_gather", f_plan)
    add("moe.gate_up", f_gu, n_act * 2 * H * F * 2)
    add("moe.down", f_dn, n_act * H * F * 2)
    add("moe.combine_norm", f_cb)


def bench_decode_pages(rows):
    """Decode attention at 16 x 8K context for several KV page sizes and head groupings (graph-replayed)."""
    from legion_b200.ops import sm100
    hbm, tf, src = peaks()
    B, D, ctx = 16, 128, 8256
    for (Hq, Hkv, page, splits) in ((32, 4, 32, 2), (32, 4, 64, 2), (32, 4, 128, 2), (32, 8, 64, 1), (64, 4, 64, 2),
                                    (32, 4, 64, 1), (32, 4, 128, 1)):
        nb = B * ((ctx + page - 1) // page)
        kc = torch.randn(nb, page, Hkv, D, device="cuda").bfloat16()
        vc = torch.randn(nb, page, Hkv, D, device="cuda").bfloat16()
        bt = torch.arange(nb, device="cuda", dtype=torch.int32).view(B, -1)
        q = torch.randn(B, Hq, D, device="cuda").bfloat16()
        cl = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
        ms = timeit_graph(lambda: sm100.paged_decode(q, kc, vc, bt, cl, D ** -0.5, n_splits=splits, max_ctx=ctx))
        byts = B * ctx * Hkv * D * 2 * 2
        rows.append(dict(kernel="paged_decode", Hq=Hq, Hkv=Hkv, page=page, splits=splits, us=ms * 1e3,
                         gbs=byts / ms / 1e6, frac_hbm=byts / ms / 1e6 / hbm, peaks=src))
        print(rows[-1], flush=True)


def bench_mla(rows):
    """Latent attention, absorbed form: decode at 16 and 64 users x 8K context with 128 heads (graph-replayed).
    FLOPs per key row = 2 * heads * (576 + 512); bytes per key row = 1152."""
    from legion_b200.ops import sm100
    hbm, tf, src = peaks()
    nh, page = 128, 64
    cases = ((16, 8192, 1), (64, 8192, 1), (1, 8192, 512))
    if CASE.get("attn"):
        cases = tuple((c[0], c[1], c[2] if len(c) > 2 else 1) for c in CASE["attn"])
    for (B, ctx, q_len) in cases:
        nb = B * ((ctx + page - 1) // page)
        cache = (torch.randn(nb, page, 1, 576, device="cuda") * 0.5).bfloat16()
        bt = torch.arange(nb, device="cuda", dtype=torch.int32).view(B, -1)
        q = (torch.randn(B * q_len, nh, 576, device="cuda") * 0.5).bfloat16()
        cu = torch.arange(0, (B + 1) * q_len, q_len, device="cuda", dtype=torch.int32)
        cl = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
        splits = sm100.mla_splits(B, q_len, nh, ctx)
        ms = timeit_graph(lambda: sm100.mla_attn(q, cache, cu, cl, bt, page, q_len, 192 ** -0.5, n_splits=splits))
        keys = B * (ctx * q_len - q_len * (q_len - 1) // 2)
        flops = 2.0 * nh * (576 + 512) * keys
        byts = B * ctx * 1152
        rows.append(dict(kernel="mla_attn", B=B, ctx=ctx, q_len=q_len, splits=splits, us=ms * 1e3,
                         tflops=flops / ms / 1e9, frac_tc=flops / ms / 1e9 / tf, gbs=byts / ms / 1e6, peaks=src))
        print(rows[-1], flush=True)


def bench_moe_fp8(rows):
    """Routed experts of a 30B-A3B-shaped layer at 16 tokens, bf16 against block-scaled FP8 weights (graph-replayed),
    plus the qkv-sized dense projection."""
    from legion_b200.ops import sm100
    from legion_b200.ops.sm100 import Fp8Weight
    hbm, tf, src = peaks()
    T, H, E, k, F = 16, 2048, 128, 8, 768
    dev = "cuda"
    x = torch.randn(T, H, device=dev).bfloat16()
    w_r = (torch.randn(E, H, device=dev) * 0.02).bfloat16()
    routing = sm100.router(x, w_r, k)
    n_act = int(torch.unique(routing.ids).numel())
    gu = (torch.randn(E, 2 * F, H, device=dev) * 0.02).bfloat16()
    dn = (torch.randn(E, H, F, device=dev) * 0.02).bfloat16()
    gq, dq = Fp8Weight.quantize(gu), Fp8Weight.quantize(dn)
    for name, a, b, bytes_per in (("bf16", gu, dn, 2), ("fp8", gq, dq, 1)):
        ms = timeit_graph(lambda: sm100.moe_experts(x, routing.ids, routing.wts, a, b, F, routing=routing))
        byts = n_act * 3 * H * F * bytes_per
        rows.append(dict(kernel="moe_experts_" + name, T=T, active_experts=n_act, us=ms * 1e3, gbs=byts / ms / 1e6,
                         frac_hbm=byts / ms / 1e6 / hbm, peaks=src))
        print(rows[-1], flush=True)
    wq = (torch.randn(5120, H, device=dev) * 0.02).bfloat16()
    wq8 = Fp8Weight.quantize(wq)
    for name, w, bytes_per in (("bf16", wq, 2), ("fp8", wq8, 1)):
        ms = timeit_graph(lambda: sm100.linear(x, w))
        byts = wq.numel() * bytes_per
        rows.append(dict(kernel="linear_5120x2048_" + name, T=T, us=ms * 1e3, gbs=byts / ms / 1e6, peaks=src))
        print(rows[-1], flush=True)


def bench_moe_nvfp4(rows):
    """Routed experts of a 30B-A3B-shaped layer at 16 tokens with the weights kept in NVFP4 (graph-replayed)."""
    from legion_b200.ops import sm100
    from legion_b200.ops.sm100 import QWeight
    hbm, tf, src = peaks()
    T, H, E, k, F = 16, 2048, 128, 8, 768
    dev = "cuda"
    x = torch.randn(T, H, device=dev).bfloat16()
    w_r = (torch.randn(E, H, device=dev) * 0.02).bfloat16()
    routing = sm100.router(x, w_r, k)
    n_act = int(torch.unique(routing.ids).numel())
    qgu = QWeight(torch.randint(0, 256, (E, 2 * F, H // 2), device=dev, dtype=torch.uint8),
                  torch.randint(48, 64, (E, 2 * F, H // 16), device=dev, dtype=torch.uint8),
                  torch.ones(2 * E, device=dev))
    qd = QWeight(torch.randint(0, 256, (E, H, F // 2), device=dev, dtype=torch.uint8),
                 torch.randint(48, 64, (E, H, F // 16), device=dev, dtype=torch.uint8), torch.ones(E, device=dev))
    ms = timeit_graph(lambda: sm100.moe_experts(x, routing.ids, routing.wts, qgu, qd, F, routing=routing))
    byts = n_act * 3 * H * F * 9 // 16
    rows.append(dict(kernel="moe_experts_nvfp4", T=T, active_experts=n_act, us=ms * 1e3, gbs=byts / ms / 1e6,
                     frac_hbm=byts / ms / 1e6 / hbm, peaks=src))
    print(rows[-1], flush=True)


def bench_moe_nv4(rows):
    """MoE block at decode size on the native NVFP4 (W4A4) path, graph-replayed, whole and by piece, for the
    30B-A3B expert shape (128 experts top-8, FFN 768) and the 80B-A3B one (512 experts top-10, FFN 512, shared
    expert stacked behind the routed ones). Bytes = the quantised bytes of the active experts (codes + scales)."""
    from legion_b200.ops import sm100
    from legion_b200.ops.sm100 import Nv4Weight
    hbm, tf, src = peaks()
    dev = "cuda"
    C = sm100.ext()
    for (name, T, H, E, k, F, shared) in (("30b-a3b", 16, 2048, 128, 8, 768, False),
                                          ("80b-a3b", 16, 2048, 512, 10, 512, True),
                                          ("80b-a3b", 64, 2048, 512, 10, 512, True),
                                          ("80b-a3b", 1, 2048, 512, 10, 512, True)):
        if CASE["tokens"] and T not in CASE["tokens"]:
            continue
        G = E + (1 if shared else 0)
        x = torch.randn(T, H, device=dev).bfloat16()
        res = torch.randn(T, H, device=dev).bfloat16()
        nw = torch.ones(H, device=dev)
        w_r = (torch.randn(E, H, device=dev) * 0.02).bfloat16()
        sh_gate = (torch.randn(1, H, device=dev) * 0.02).bfloat16() if shared else None

        def rand_w(rows_, K):
            codes = torch.randint(0, 256, (G, rows_, K // 2), device=dev, dtype=torch.uint8)
            lin = torch.randint(48, 64, (G * rows_, K // 16), device=dev, dtype=torch.uint8)
            atoms = torch.zeros(C.nv4_sf_bytes(G * rows_, K), dtype=torch.uint8, device=dev)
            C.nv4_pack_scales(lin, atoms)
            return codes, atoms
        gc, gs = rand_w(2 * F, H)
        dc, ds = rand_w(H, F)
        qgu = Nv4Weight(gc, gs, torch.full((2 * G,), 1e-3, device=dev))
        qdn = Nv4Weight(dc, ds, torch.full((G,), 1e-3, device=dev))
        kw = dict(shared_slot=shared, sh_gate=sh_gate, slot_stride=128)
        routing = sm100.router(x, w_r, k, **kw)
        n_act = int(torch.unique(routing.ids).numel()) + (1 if shared else 0)
        byts = n_act * 3 * H * F * 9 // 16

        def block():
            xq = sm100.nv4_quant_act(x, norm=(nw, 1e-6, 0.0), residual=res, want_normed=True, key="bench_x")
            r = sm100.router(xq.normed, w_r, k, **kw)
            return sm100._moe_experts_nv4(xq.normed, r.ids, r.wts, qgu, qdn, F, 0, None, None, xq.summed, None,
                                          (nw, 1e-6, 0.0), r, xq=xq)

        def add(part, fn, b=0):
            ms = timeit_graph(fn)
            rows.append(dict(kernel="moe_nv4", shape=name, T=T, part=part, active=n_act, us=ms * 1e3,
                             gbs=b / ms / 1e6 if b else 0.0, frac_hbm=b / ms / 1e6 / hbm if b else 0.0, peaks=src))
            print(rows[-1], flush=True)
        add("block(addnorm+quant, route, gate_up, down, combine+norm)", block, byts)
        xq = sm100.nv4_quant_act(x, key="bench_x2")
        ws = sm100.Workspace.get(torch.device(dev))
        dr = routing.dense
        hs = torch.tensor([32.0 / 2688.0], device=dev)
        rows_h = dr.n_slots * dr.stride
        hq = torch.zeros(rows_h, F // 2, dtype=torch.uint8, device=dev)
        hsf = torch.zeros(C.nv4_sf_bytes(rows_h, F), dtype=torch.uint8, device=dev)
        y = torch.zeros(T * k + 64, H, dtype=torch.bfloat16, device=dev)
        add("addnorm_quant", lambda: sm100.nv4_quant_act(x, norm=(nw, 1e-6, 0.0), residual=res, want_normed=True,
                                                         key="bench_x3"))
        add("route", lambda: sm100.router(x, w_r, k, **kw), w_r.numel() * 2)
        add("gate_up", lambda: C.wgemm_nv4(qgu.view2d(), qgu.sf, qgu.gscale, xq.codes, xq.sf, xq.gscale, 1, None, None,
                                           None, None, F, True, F, 0, dr.bn, ws.status, dr.tile_group, dr.zeros,
                                           dr.tile_ntok, dr.meta, dr.n_slots, 2 * F, 0, dr.slot_base, hq, hsf, hs),
            n_act * 2 * H * F * 9 // 16)
        add("down", lambda: C.wgemm_nv4(qdn.view2d(), qdn.sf, qdn.gscale, hq, hsf, hs, 0, y, None, dr.tok_scale,
                                        dr.out_rows, H, False, 0, 0, dr.bn, ws.status, dr.tile_group, dr.slot_base,
                                        dr.tile_ntok, dr.meta, dr.n_slots, H, 0, None, None, None, None),
            n_act * H * F * 9 // 16)


def bench_gdn(rows):
    """Gated DeltaNet recurrence over a prompt (80B-A3B hybrid shape: 16 key / 32 value heads of dim 128) and over a
    decode step of 16 sequences: tokens per second of the state update."""
    from legion_b200.ops import sm100
    hbm, tf, src = peaks()
    nk, nv, dk, dv = 16, 32, 128, 128
    C = 2 * nk * dk + nv * dv
    for n_seq, L in (CASE["attn"] or ((1, 8192), (16, 1))):
        T = n_seq * L
        qkv = (torch.randn(T, C, device="cuda") * 0.3).bfloat16()
        g = -torch.rand(T, nv, device="cuda") * 0.1
        beta = torch.rand(T, nv, device="cuda")
        state = torch.zeros(n_seq, nv, dk, dv, device="cuda")
        cu = torch.arange(0, (n_seq + 1) * L, L, device="cuda", dtype=torch.int32)
        slots = torch.arange(n_seq, device="cuda", dtype=torch.int32)
        cu_host = list(range(0, (n_seq + 1) * L, L))
        ms = timeit(lambda: sm100.gdn_recurrent(qkv, g, beta, state, cu, slots, nk, nv, dk, dv, False, dk ** -0.5,
                                                cu_host=cu_host), iters=5, flush=False)
        # prompts of >= 64 tokens run the chunked tensor-core scan (prep + scan kernels), decode rows the
        # state-streaming kernel. Chunk-form FLOPs per 64-token chunk and head: K K^T, Q K^T, T V, T K (prep) and
        # W S, Q' S, M D, D^T K' (scan), each 2 * 64 * 64 * 128 or 2 * 64 * 128 * 128
        row = dict(kernel="gdn (chunked scan)" if L >= 64 else "gdn_recurrent", n_seq=n_seq, L=L, ms=ms,
                   tok_s=T / ms * 1e3, state_gbs=n_seq * nv * dk * dv * 4 * 2 / ms / 1e6, peaks=src)
        if L >= 64:
            chunks = n_seq * ((L + 63) // 64) * nv
            flops = chunks * (4 * 2 * 64 * 64 * 128 + 4 * 2 * 64 * 128 * 128)
            row["tflops"] = flops / ms / 1e9
        rows.append(row)
        print(rows[-1], flush=True)


def bench_gemm(rows):
    from legion_b200.ops import sm100
    hbm, tf, src = peaks()
    for (T, N, K) in CASE["gemm"] or [(8192, 5120, 2048), (8192, 2048, 4096), (4096, 8192, 8192), (16, 5120, 2048), (16, 2048, 4096),
                      (64, 151936, 2048), (1, 5120, 2048), (256, 17408, 5120)]:
        x = torch.randn(T, K, device="cuda").bfloat16()
        w = torch.randn(N, K, device="cuda").bfloat16()
        out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        ms = timeit(lambda: sm100.linear(x, w, out=out))
        ms_t = timeit(lambda: torch.matmul(x, w.t(), out=out))
        fl = 2.0 * T * N * K / ms / 1e9
        gb = (N * K + T * K + T * N) * 2 / ms / 1e6
        rows.append(dict(kernel="wgemm", T=T, N=N, K=K, ms=ms, tflops=fl, gbs=gb, frac_tflops=fl / tf, frac_hbm=gb / hbm,
                         cublas_ms=ms_t, peaks=src))
        print(rows[-1], flush=True)


def bench_moe(rows):
    from legion_b200.ops import sm100
    hbm, tf, src = peaks()
    E, k, H, F = 128, 8, 2048, 768
    wgu = (torch.randn(E, 2 * F, H, device="cuda") * 0.02).bfloat16()
    wd = (torch.randn(E, H, F, device="cuda") * 0.02).bfloat16()
    for T in (CASE["tokens"] or (1, 16, 64, 1024, 8192)):
        x = torch.randn(T, H, device="cuda").bfloat16()
        logits = torch.randn(T, E, device="cuda")
        ids, wts = sm100.router_topk(logits, k)
        ms = timeit(lambda: sm100.moe_experts(x, ids, wts, wgu, wd, F))
        n_act = int(torch.unique(ids).numel())
        byts = n_act * 3 * H * F * 2
        fl = 2.0 * T * k * 3 * H * F / ms / 1e9
        rows.append(dict(kernel="moe_experts", T=T, active_experts=n_act, ms=ms, tflops=fl, weight_gbs=byts / ms / 1e6,
                         frac_tflops=fl / tf, frac_hbm=byts / ms / 1e6 / hbm, peaks=src))
        print(rows[-1], flush=True)


def bench_decode_attn(rows):
    from legion_b200.ops import sm100
    hbm, tf, src = peaks()
    Hq, Hkv, D, page = 32, 4, 128, 64
    for B, ctx in (CASE["attn"] or ((1, 8192), (16, 8192), (64, 8192), (16, 1024))):
        nb = B * ((ctx + page - 1) // page)
        kc = torch.randn(nb, page, Hkv, D, device="cuda").bfloat16()
        vc = torch.randn(nb, page, Hkv, D, device="cuda").bfloat16()
        bt = torch.arange(nb, device="cuda", dtype=torch.int32).view(B, -1)
        q = torch.randn(B, Hq, D, device="cuda").bfloat16()
        cl = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
        ms = timeit(lambda: sm100.paged_decode(q, kc, vc, bt, cl, D ** -0.5, max_ctx=ctx))
        byts = B * ctx * Hkv * D * 2 * 2
        rows.append(dict(kernel="paged_decode", B=B, ctx=ctx, ms=ms, gbs=byts / ms / 1e6, frac_hbm=byts / ms / 1e6 / hbm,
                         peaks=src))
        print(rows[-1], flush=True)


def bench_prefill_attn(rows):
    from legion_b200.ops import sm100
    hbm, tf, src = peaks()
    Hq, Hkv, D, page = CASE.get("heads") or (32, 4, 128, 64)
    for n_seq, L in (CASE["attn"] or ((1, 8192), (4, 2048), (1, 32768))):
        nb = n_seq * (L // page)
        kc = torch.randn(nb, page, Hkv, D, device="cuda").bfloat16()
        vc = torch.randn(nb, page, Hkv, D, device="cuda").bfloat16()
        bt = torch.arange(nb, device="cuda", dtype=torch.int32).view(n_seq, -1)
        q = torch.randn(n_seq * L, Hq, D, device="cuda").bfloat16()
        cu = torch.arange(0, (n_seq + 1) * L, L, device="cuda", dtype=torch.int32)
        cl = torch.full((n_seq,), L, device="cuda", dtype=torch.int32)
        out = torch.empty_like(q)
        ms = timeit(lambda: sm100.prefill_attn(q, kc, vc, cu, cl, bt, L, D ** -0.5, out=out), iters=5)
        fl = 4.0 * n_seq * L * L / 2 * D * Hq / ms / 1e9
        rows.append(dict(kernel="prefill_attn", n_seq=n_seq, L=L, heads=(Hq, Hkv, D), ms=ms, tflops=fl,
                         frac_tflops=fl / tf, peaks=src))
        print(rows[-1], flush=True)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="gemm,moe,decode_attn,prefill_attn")
    ap.add_argument("--json", default=None)
    ap.add_argument("--tokens", default=None, help="moe: comma list of token counts")
    ap.add_argument("--attn", default=None, help="attention: BxCTX[,BxCTX...] (decode) or SEQSxLEN (prefill)")
    ap.add_argument("--gemm", default=None, help="gemm: TxNxK[,TxNxK...]")
    ap.add_argument("--heads", default=None, help="prefill attention: HQxHKVxD (page 64), default 32x4x128")
    ap.add_argument("--iters", type=int, default=None)
    ap.add_argument("--warmup-iters", type=int, default=None)
    a = ap.parse_args(argv)
    ITERS["iters"], ITERS["warmup"] = a.iters, a.warmup_iters
    if a.tokens:
        CASE["tokens"] = tuple(int(x) for x in a.tokens.split(","))
    if a.attn:
        CASE["attn"] = tuple(tuple(int(y) for y in x.split("x")) for x in a.attn.split(","))
    if a.heads:
        hq, hkv, d = (int(x) for x in a.heads.split("x"))
        CASE["heads"] = (hq, hkv, d, 64)
    if a.gemm:
        CASE["gemm"] = [tuple(int(y) for y in x.split("x")) for x in a.gemm.split(",")]
    rows = []
    table = {"moe_nv4": bench_moe_nv4, "gdn": bench_gdn, "moe_fp8": bench_moe_fp8, "mla": bench_mla, "moe_nvfp4": bench_moe_nvfp4, "layer_parts": bench_layer_parts, "decode_pages": bench_decode_pages, "gemm": bench_gemm, "moe": bench_moe, "decode_attn": bench_decode_attn, "prefill_attn": bench_prefill_attn}
    for name in a.only.split(","):
        table[name](rows)
    from legion_b200.ops.sm100 import Workspace
    torch.cuda.synchronize()
    print("status word:", Workspace.get("cuda").check())
    if a.json:
        json.dump(rows, open(a.json, "w"), indent=1)


if __name__ == "__main__":
    main(sys.argv[1:])
