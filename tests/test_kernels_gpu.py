"""sm_100a kernels against the fp32 PyTorch reference of the same op (small, ragged and boundary shapes)."""
import math

import pytest
import torch

from legion_b200.ops import reference as ref

pytestmark = pytest.mark.gpu

DEV = "cuda"


def sm():
    from legion_b200.ops import sm100
    return sm100


def status_ok():
    from legion_b200.ops.sm100 import Workspace
    torch.cuda.synchronize()
    assert Workspace.get(torch.device(DEV)).check() == 0


def close(a, b, rtol=2e-2, atol=2e-2):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4g} (ref max {b.abs().max().item():.4g})"


def rnd(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).bfloat16()


@pytest.mark.parametrize("T,N,K", [(1, 128, 64), (16, 256, 128), (33, 200, 192), (100, 384, 2048), (300, 130, 72),
                                   (16, 5120, 2048), (513, 512, 256)])
@pytest.mark.parametrize("split_k", [1, 3])
def test_linear(T, N, K, split_k):
    torch.manual_seed(T * 7 + N)
    x, w = rnd(T, K), rnd(N, K, scale=K ** -0.5)
    out = sm().linear(x, w, split_k=split_k)
    status_ok()
    close(out, ref.linear(x, w))


def test_linear_structured_identity():
    # one-hot rows localise layout bugs: out[t, n] must be exactly w[n, t]
    K = 128
    x = torch.eye(K, device=DEV).bfloat16()
    w = rnd(256, K)
    out = sm().linear(x, w, split_k=1)
    status_ok()
    assert torch.equal(out, w.t().contiguous())


def test_linear_residual_f32_and_repeat():
    x, w, r = rnd(40, 256), rnd(384, 256, scale=1 / 16), rnd(40, 384)
    a = sm().linear(x, w, residual=r)
    b = sm().linear(x, w, residual=r)
    status_ok()
    close(a, ref.linear(x, w, residual=r))
    assert torch.equal(a, b)  # run-to-run determinism
    f = sm().linear(x, w, out_dtype=torch.float32)
    close(f, ref.linear(x, w, out_dtype=torch.float32), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("T,F,K,split_k", [(5, 128, 64, 1), (64, 768, 2048, 1), (130, 200, 256, 1), (16, 768, 2048, 4)])
def test_gate_up_act(T, F, K, split_k):
    x, w = rnd(T, K), rnd(2 * F, K, scale=K ** -0.5)
    out = sm().gate_up_act(x, w, F, split_k=split_k)
    status_ok()
    close(out, ref.gate_up_act(x, w, F))


@pytest.mark.parametrize("T,E,k,H,F", [(4, 8, 2, 256, 128), (16, 128, 8, 512, 256), (300, 16, 4, 256, 192), (1, 8, 2, 128, 64)])
def test_moe_experts(T, E, k, H, F):
    torch.manual_seed(E + T)
    x = rnd(T, H)
    logits = torch.randn(T, E, device=DEV)
    ids, wts = sm().router_topk(logits, k)
    rids, rwts = ref.router_topk(logits, k)
    assert torch.equal(ids.cpu(), rids.cpu())
    close(wts, rwts, 1e-4, 1e-5)
    wgu, wd = rnd(E, 2 * F, H, scale=H ** -0.5), rnd(E, H, F, scale=F ** -0.5)
    res = rnd(T, H)
    out = sm().moe_experts(x, ids, wts, wgu, wd, F, residual=res)
    status_ok()
    want = ref.moe_experts(x, ids, wts, wgu, wd, F) + res.float()
    close(out, want, 3e-2, 3e-2)
    out2 = sm().moe_experts(x, ids, wts, wgu, wd, F, residual=res)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("T,E,k,e_lo,n_local", [(1, 128, 8, 0, 128), (16, 128, 8, 0, 128), (100, 64, 6, 16, 32),
                                                  (128, 8, 8, 0, 8)])
def test_moe_plan_fused_equals_three_pass(T, E, k, e_lo, n_local):
    """The single-launch plan + gather of decode-sized steps gives the same plan and rows as count/scan/fill/gather."""
    from legion_b200.ops.sm100 import MoePlan, ext
    C = ext()
    H, bn = 256, 32
    x = rnd(T, H)
    ids, wts = sm().router_topk(torch.randn(T, E, device=DEV), k)
    a, b = MoePlan(T, k, n_local, bn, DEV), MoePlan(T, k, n_local, bn, DEV)
    xa = torch.zeros(T * k + bn, H, dtype=torch.bfloat16, device=DEV)
    xb = torch.zeros_like(xa)
    C.moe_plan(ids, wts, e_lo, n_local, bn, a.counts, a.offsets, a.sorted_token, a.sorted_pair, a.sorted_w,
               a.tile_group, a.tile_tok0, a.tile_ntok, a.meta)
    C.gather_rows(x, a.sorted_token, a.meta[1:2], xa[:T * k])
    C.moe_plan_gather(ids, wts, e_lo, n_local, bn, b.counts, b.offsets, b.sorted_token, b.sorted_pair, b.sorted_w,
                      b.tile_group, b.tile_tok0, b.tile_ntok, b.meta, x, xb)
    n_tiles, n_rows = a.meta.tolist()
    assert b.meta.tolist() == [n_tiles, n_rows]
    assert torch.equal(a.counts, b.counts) and torch.equal(a.offsets, b.offsets)
    for name in ("sorted_token", "sorted_pair", "sorted_w"):
        assert torch.equal(getattr(a, name)[:n_rows], getattr(b, name)[:n_rows]), name
    for name in ("tile_group", "tile_tok0", "tile_ntok"):
        assert torch.equal(getattr(a, name)[:n_tiles], getattr(b, name)[:n_tiles]), name
    assert torch.equal(xa, xb)


@pytest.mark.parametrize("T,E,k,H,mode", [(1, 128, 8, 2048, "softmax"), (16, 128, 8, 2048, "softmax"),
                                          (37, 256, 8, 512, "sigmoid"), (64, 8, 2, 256, "softmax"),
                                          (16, 256, 8, 7168, "sigmoid"), (33, 64, 6, 4096, "softmax")])
def test_router_fused(T, E, k, H, mode):
    """One-launch router (logits + top-k) against fp32 logits and the reference selection; hidden widths from 4096
    on split the columns over CTAs and add the partial logits in a fixed order."""
    torch.manual_seed(T + E)
    x, w = rnd(T, H), rnd(E, H, scale=H ** -0.5)
    bias = torch.randn(E, device=DEV) * 0.05 if mode == "sigmoid" else None
    kw = dict(mode=mode, renorm=True, route_scale=1.5, bias=bias)
    if mode == "sigmoid":
        kw.update(n_group=8, topk_group=4)
    for _ in range(2):      # the done counter must be left ready for the next call
        routing = sm().router(x, w, k, **kw)
    ids, wts = routing
    assert routing.dense is not None
    logits = x.float() @ w.float().t()
    rids, rwts = ref.router_topk(logits, k, **kw)
    # near-ties may swap under a different summation order: compare as sets through the gathered logits
    same = (ids.cpu().sort(1).values == rids.cpu().sort(1).values).all(1)
    assert same.float().mean() >= 0.95
    rows = same.nonzero().flatten()
    o1, o2 = ids.cpu()[rows].sort(1).indices, rids.cpu()[rows].sort(1).indices
    close(wts.cpu()[rows].gather(1, o1), rwts.cpu()[rows].gather(1, o2), 2e-3, 1e-4)


@pytest.mark.parametrize("T,E,k,H,F", [(1, 128, 8, 512, 256), (16, 128, 8, 2048, 768), (33, 16, 4, 256, 192),
                                       (64, 8, 2, 256, 128), (16, 32, 4, 4096, 256)])
def test_moe_dense_route(T, E, k, H, F):
    """Decode-sized path: norm + router + top-k + dense tables in one launch, expert GEMMs without a gather."""
    torch.manual_seed(T * 3 + E)
    hidden, res = rnd(T, H), rnd(T, H)
    nw = torch.rand(H, device=DEV) + 0.5
    w_r = rnd(E, H, scale=H ** -0.5)
    wgu, wd = rnd(E, 2 * F, H, scale=H ** -0.5), rnd(E, H, F, scale=F ** -0.5)
    r = sm().router(hidden, w_r, k, norm=(nw, 1e-6, 0.0))
    want_x, _ = ref.rmsnorm(hidden, nw, 1e-6, 0.0)
    close(r.x_normed, want_x, 1e-2, 1e-2)
    x = r.x_normed
    out = sm().moe_experts(x, r.ids, r.wts, wgu, wd, F, residual=res, routing=r)
    status_ok()
    want = ref.moe_experts(x, r.ids, r.wts, wgu, wd, F) + res.float()
    close(out, want, 3e-2, 3e-2)
    plan_path = sm().moe_experts(x, r.ids, r.wts, wgu, wd, F, residual=res)       # gather path, same routing
    close(out, plan_path, 1e-2, 1e-2)
    n_act = int(torch.unique(r.ids).numel())
    assert r.dense.meta.tolist() == [n_act, n_act * r.dense.bn]
    out2 = sm().moe_experts(x, r.ids, r.wts, wgu, wd, F, residual=res, routing=r)
    assert torch.equal(out, out2)


def test_moe_combine_with_norm():
    T, E, k, H, F = 16, 32, 4, 512, 128
    x = rnd(T, H)
    ids, wts = sm().router_topk(torch.randn(T, E, device=DEV), k)
    wgu, wd = rnd(E, 2 * F, H, scale=H ** -0.5), rnd(E, H, F, scale=F ** -0.5)
    res = rnd(T, H)
    nw = torch.rand(H, device=DEV) + 0.5
    out, normed = sm().moe_experts(x, ids, wts, wgu, wd, F, residual=res, norm=(nw, 1e-6, 0.0))
    plain = sm().moe_experts(x, ids, wts, wgu, wd, F, residual=res)
    status_ok()
    assert torch.equal(out, plain)
    want, _ = ref.rmsnorm(out, nw, 1e-6, 0.0)
    close(normed, want, 2e-2, 2e-2)


def test_router_group_limited():
    T, E = 37, 256
    logits = torch.randn(T, E, device=DEV)
    bias = torch.randn(E, device=DEV) * 0.1
    ids, wts = sm().router_topk(logits, 8, mode="sigmoid", renorm=True, route_scale=2.5, bias=bias, n_group=8, topk_group=4)
    rids, rwts = ref.router_topk(logits, 8, mode="sigmoid", renorm=True, route_scale=2.5, bias=bias, n_group=8, topk_group=4)
    assert torch.equal(ids.cpu(), rids.cpu())
    close(wts, rwts, 1e-4, 1e-5)


@pytest.mark.parametrize("H", [256, 2048, 5120])
def test_rmsnorm(H):
    x, r = rnd(19, H), rnd(19, H)
    w = torch.rand(H, device=DEV) + 0.5
    y, s = sm().rmsnorm(x, w, 1e-6, residual=r)
    ry, rs = ref.rmsnorm(x, w, 1e-6, residual=r)
    close(y, ry)
    assert torch.equal(s, rs)
    y2, _ = sm().rmsnorm(x, w, 1e-6, w_offset=1.0)
    close(y2, ref.rmsnorm(x, w, 1e-6, w_offset=1.0)[0])


def make_cache(n_blocks, page, Hkv, D):
    return rnd(n_blocks, page, Hkv, D), rnd(n_blocks, page, Hkv, D)


@pytest.mark.parametrize("D,Hq,Hkv,rot,gated", [(128, 8, 2, 128, False), (64, 4, 2, 64, False), (256, 4, 1, 64, True)])
def test_qk_norm_rope_append(D, Hq, Hkv, rot, gated):
    T, page, n_blocks = 21, 16, 8
    qw = Hq * D * (2 if gated else 1)
    qkv = rnd(T, qw + 2 * Hkv * D)
    qn, kn = torch.rand(D, device=DEV) + 0.5, torch.rand(D, device=DEV) + 0.5
    cs = ref.rope_cos_sin(512, rot, 1e6, device=DEV)
    pos = torch.arange(100, 100 + T, device=DEV, dtype=torch.int32)
    slots = torch.randperm(n_blocks * page, device=DEV)[:T].long()
    kc, vc = make_cache(n_blocks, page, Hkv, D)
    kc2, vc2 = kc.clone(), vc.clone()
    q = sm().qk_norm_rope_append(qkv, Hq, Hkv, D, qn, kn, 1e-6, 0.0, cs, rot, pos, slots, kc, vc, gated_q=gated)
    rq, rgate = ref.qk_norm_rope_append(qkv, Hq, Hkv, D, qn, kn, 1e-6, 0.0, cs, rot, pos, slots, kc2, vc2, gated_q=gated)
    close(q, rq)
    close(kc, kc2)
    assert torch.equal(vc, vc2)
    if gated:
        attn = rnd(T, Hq, D)
        g = sm().sigmoid_gate(attn, qkv, Hq, D)
        close(g, attn.float() * torch.sigmoid(rgate.float()))


@pytest.mark.parametrize("D,Hq,Hkv,page", [(128, 32, 4, 64), (64, 4, 2, 16), (256, 16, 2, 64), (128, 40, 8, 16), (128, 6, 2, 32)])
def test_paged_decode(D, Hq, Hkv, page):
    torch.manual_seed(D + Hq)
    B = 3
    ctx = [1, 77, 300]
    n_blocks = 64
    kc, vc = make_cache(n_blocks, page, Hkv, D)
    width = (max(ctx) + page - 1) // page
    bt = torch.stack([torch.randperm(n_blocks, device=DEV)[:width] for _ in range(B)]).int()
    q = rnd(B, Hq, D)
    ctx_t = torch.tensor(ctx, device=DEV, dtype=torch.int32)
    scale = D ** -0.5
    want = ref.paged_attention(q, kc, vc, bt, ctx_t, torch.arange(B + 1), scale)
    wantw = ref.paged_attention(q, kc, vc, bt, ctx_t, torch.arange(B + 1), scale, window=50)
    for impl in ("tc", "simt"):
        for ns in (1, 3):
            out = sm().paged_decode(q, kc, vc, bt, ctx_t, scale, n_splits=ns, impl=impl)
            status_ok()
            close(out, want)
        outw = sm().paged_decode(q, kc, vc, bt, ctx_t, scale, window=50, n_splits=2, impl=impl)
        status_ok()
        close(outw, wantw)


@pytest.mark.parametrize("D,Hq,Hkv,page", [(128, 4, 2, 64), (64, 4, 2, 16), (256, 2, 1, 64), (128, 8, 8, 32)])
def test_prefill_attn(D, Hq, Hkv, page):
    torch.manual_seed(D + page)
    q_lens = [5, 130, 257]
    ctx = [5, 200, 257]          # second sequence has 70 cached tokens before its chunk
    n_blocks = 48
    kc, vc = make_cache(n_blocks, page, Hkv, D)
    width = (max(ctx) + page - 1) // page + 1
    bt = torch.stack([torch.randperm(n_blocks, device=DEV)[:width] for _ in q_lens]).int()
    cu = torch.tensor([0, 5, 135, 392], device=DEV, dtype=torch.int32)
    q = rnd(392, Hq, D)
    ctx_t = torch.tensor(ctx, device=DEV, dtype=torch.int32)
    scale = D ** -0.5
    out = sm().prefill_attn(q, kc, vc, cu, ctx_t, bt, max(q_lens), scale)
    status_ok()
    want = ref.paged_attention(q, kc, vc, bt, ctx_t, cu, scale)
    close(out, want, 3e-2, 3e-2)
    outw = sm().prefill_attn(q, kc, vc, cu, ctx_t, bt, max(q_lens), scale, window=64)
    status_ok()
    close(outw, ref.paged_attention(q, kc, vc, bt, ctx_t, cu, scale, window=64), 3e-2, 3e-2)


def test_argmax_and_sample():
    V = 151936
    logits = torch.randn(5, V, device=DEV)
    logits[2, 77] = 50.0
    logits[3, V - 1] = 60.0
    assert torch.equal(sm().argmax(logits).cpu(), ref.argmax(logits).cpu())
    assert torch.equal(sm().argmax(logits.bfloat16()).cpu(), ref.argmax(logits.bfloat16()).cpu())
    temp = torch.tensor([0.0, 1.0, 1.0, 0.7, 1.0], device=DEV)
    tk = torch.tensor([0, 1, 50, 0, 0], device=DEV, dtype=torch.int32)
    tp = torch.tensor([1.0, 1.0, 1.0, 0.5, 1.0], device=DEV)
    mp = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0], device=DEV)
    seeds = torch.arange(5, device=DEV, dtype=torch.int64) + 1234
    steps = torch.zeros(5, device=DEV, dtype=torch.int32)
    out = sm().sample(logits, temp, tk, tp, mp, seeds, steps).cpu()
    am = ref.argmax(logits).cpu()
    assert out[0] == am[0] and out[1] == am[1] and out[2] == 77 and out[3] == V - 1
    # unrestricted row: empirical distribution over a tiny vocab matches softmax
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0]], device=DEV).repeat(4000, 1)
    t1 = torch.ones(4000, device=DEV)
    sd = torch.arange(4000, device=DEV, dtype=torch.int64)
    draws = sm().sample(small, t1, None, None, None, sd, None).cpu()
    freq = torch.bincount(draws, minlength=4).float() / 4000
    close(freq, torch.softmax(small[0].cpu(), -1), 0.0, 0.03)


@pytest.mark.parametrize("nk,nv,dk,dv,tiled", [(2, 4, 64, 64, False), (2, 4, 128, 128, True), (4, 4, 32, 32, False)])
def test_gdn(nk, nv, dk, dv, tiled):
    torch.manual_seed(dk)
    cu = torch.tensor([0, 1, 9, 40], device=DEV, dtype=torch.int32)
    slots = torch.tensor([2, 0, 3], device=DEV, dtype=torch.int32)
    T = 40
    C = 2 * nk * dk + nv * dv
    x = rnd(T, C)
    w = torch.randn(C, 4, device=DEV) * 0.5
    cst = torch.randn(4, C, 3, device=DEV)
    cst2 = cst.clone()
    y = sm().causal_conv1d_silu(x, w, None, cst, cu, slots)
    ry = ref.causal_conv1d_silu(x, w, None, cst2, cu, slots)
    close(y, ry)
    close(cst, cst2, 1e-5, 1e-5)
    a, b = rnd(T, nv), rnd(T, nv)
    A = -torch.rand(nv, device=DEV) - 0.1
    dtb = torch.randn(nv, device=DEV)
    g, beta = sm().gdn_gates(a, b, A, dtb)
    rg, rb = ref.gdn_gates(a, b, A, dtb)
    close(g, rg, 1e-4, 1e-5)
    close(beta, rb, 1e-4, 1e-5)
    st = torch.randn(4, nv, dk, dv, device=DEV) * 0.1
    st2 = st.clone()
    o = sm().gdn_recurrent(y, g, beta, st, cu, slots, nk, nv, dk, dv, tiled, dk ** -0.5)
    ro = ref.gdn_recurrent(ry, rg, rb, st2, cu, slots, nk, nv, dk, dv, tiled, dk ** -0.5)
    close(o, ro, 3e-2, 3e-2)
    close(st, st2, 2e-2, 2e-2)
    z = rnd(T, nv * dv)
    nw = torch.rand(dv, device=DEV) + 0.5
    n = sm().gated_rmsnorm(o, z, nw, 1e-6)
    close(n, ref.gated_rmsnorm(o, z.view(T, nv, dv), nw, 1e-6))


def test_block_formats_roundtrip():
    from legion_b200.ops.sm100 import ext
    C = ext()
    w = rnd(256, 512, scale=0.02)
    gs = torch.tensor([float(w.float().abs().max()) / (6 * 448)], device=DEV)
    codes = torch.empty(256, 256, dtype=torch.uint8, device=DEV)
    scales = torch.empty(256, 32, dtype=torch.uint8, device=DEV)
    C.nvfp4_quant(w, gs, codes, scales)
    back = torch.empty_like(w)
    C.nvfp4_dequant(codes, scales, gs, back)
    rel = (back.float() - w.float()).norm() / w.float().norm()
    assert rel < 0.12, rel
    q8 = torch.empty(256, 512, dtype=torch.uint8, device=DEV)
    sc = torch.empty(2, 4, dtype=torch.float32, device=DEV)
    C.fp8_block_quant(w, 128, 128, q8, sc)
    back8 = torch.empty_like(w)
    C.fp8_block_dequant(q8, sc, 128, 128, back8)
    rel8 = (back8.float() - w.float()).norm() / w.float().norm()
    assert rel8 < 0.04, rel8
    want = (q8.view(torch.float8_e4m3fn).float().view(2, 128, 4, 128) * sc[:, None, :, None]).view(256, 512)
    close(back8, want, 1e-2, 1e-6)


def test_wait_deadline_sets_status_and_context_survives():
    from legion_b200.ops.sm100 import ext
    C = ext()
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    C.wait_flag(flag, 1, 2_000_000, status)  # 2 ms deadline on a flag nothing sets
    torch.cuda.synchronize()
    assert int(status.item()) == 5
    assert float((torch.ones(4, device=DEV) * 2).sum()) == 8.0


def test_token_logprobs_and_spec_accept():
    torch.manual_seed(5)
    R, V, n = 7, 151936, 5
    logits = torch.randn(R, V, device=DEV) * 3
    chosen = torch.randint(0, V, (R,), device=DEV, dtype=torch.int32)
    lp, ids, tl = sm().token_logprobs(logits, chosen, n)
    ref_lp = torch.log_softmax(logits.double(), -1)
    close(lp, ref_lp.gather(1, chosen.long()[:, None])[:, 0], 1e-4, 1e-4)
    tv, ti = ref_lp.topk(n, -1)
    assert torch.equal(ids.long().cpu(), ti.cpu())
    close(tl, tv, 1e-4, 1e-4)
    # greedy acceptance: 3 sequences with 4, 2 and 0 drafts
    cu = torch.tensor([0, 5, 8, 9], device=DEV, dtype=torch.int32)
    target = torch.tensor([11, 12, 13, 99, 15, 21, 22, 23, 31], device=DEV, dtype=torch.int32)
    draft = torch.tensor([[11, 12, 13, 14], [21, 22, 0, 0], [0, 0, 0, 0]], device=DEV, dtype=torch.int32)
    nd = torch.tensor([4, 2, 0], device=DEV, dtype=torch.int32)
    acc, bonus, rej = sm().spec_accept(target, cu, draft, nd)
    assert acc.tolist() == [3, 2, 0] and bonus.tolist() == [99, 23, 31] and int(rej.item()) == 1


@pytest.mark.parametrize("tname", ["Q8_0", "Q4_0", "Q4_K", "Q5_K", "Q6_K", "IQ4_NL"])
def test_gguf_dequant_kernel_matches_host(tname):
    """Random block bytes (with sane fp16 scales) expand to the same values on the device as in numpy."""
    import numpy as np
    from legion_b200.loaders.gguf import GGML_TYPES, TYPE_ID, dequantize
    from legion_b200.ops.sm100 import ext
    tid = TYPE_ID[tname]
    _, be, bb = GGML_TYPES[tid]
    n_blocks = 64 * (256 // be)
    rng = np.random.default_rng(3)
    raw = rng.integers(0, 256, size=(n_blocks, bb), dtype=np.uint8)
    scale = (rng.random(n_blocks) * 0.1 + 0.01).astype(np.float16).view(np.uint8).reshape(-1, 2)
    if tname in ("Q8_0", "Q4_0", "IQ4_NL"):
        raw[:, 0:2] = scale
    elif tname in ("Q4_K", "Q5_K"):
        raw[:, 0:2] = scale
        raw[:, 2:4] = scale[::-1]
    else:
        raw[:, 208:210] = scale
    shape = (n_blocks * be // 256, 256)
    want = dequantize(raw.reshape(-1), tid, shape)
    out = torch.empty(shape, dtype=torch.bfloat16, device=DEV)
    ext().gguf_dequant(torch.from_numpy(raw.reshape(-1).copy()).to(DEV), tid, out)
    close(out, torch.from_numpy(want).bfloat16(), 1e-2, 1e-3)


@pytest.mark.parametrize("T,N,K,split_k", [(1, 128, 256, 1), (16, 384, 512, 1), (16, 384, 1024, 3), (300, 256, 768, 1),
                                            (40, 5120, 2048, None)])
def test_linear_nvfp4_weights(T, N, K, split_k):
    """GEMM over weights kept in NVFP4 (expanded to bf16 operand tiles inside the kernel) against the fp32 product
    with the de-quantised weights."""
    from legion_b200.ops.sm100 import QWeight
    torch.manual_seed(T + N)
    x = rnd(T, K)
    w = rnd(N, K, scale=K ** -0.5)
    qw = QWeight.quantize(w)
    deq = qw.dequantize()
    assert (deq.float() - w.float()).abs().max() < 0.3 * w.float().abs().max()      # sanity of the encoding itself
    out = sm().linear(x, qw, split_k=split_k)
    status_ok()
    close(out, ref.linear(x, deq))
    res = rnd(T, N)
    out = sm().linear(x, qw, residual=res, split_k=split_k)
    close(out, ref.linear(x, deq).float() + res.float())


def test_moe_nvfp4_weights():
    from legion_b200.ops.sm100 import QWeight
    torch.manual_seed(11)
    E, k, H, F = 16, 4, 512, 256
    wgu, wd = rnd(E, 2 * F, H, scale=H ** -0.5), rnd(E, H, F, scale=F ** -0.5)
    qgu, qd = QWeight.quantize(wgu, dual_rows=F), QWeight.quantize(wd)
    dgu, dd = qgu.dequantize(), qd.dequantize()
    x1 = rnd(7, H)
    close(sm().gate_up_act(x1, QWeight(qgu.codes[0], qgu.scales[0], qgu.gscale[:2]), F), ref.gate_up_act(x1, dgu[0], F))
    for T in (16, 200):                       # dense-routing path and plan + gather path
        x = rnd(T, H)
        w_r = rnd(E, H, scale=H ** -0.5)
        r = sm().router(x, w_r, k)
        out = sm().moe_experts(x, r.ids, r.wts, qgu, qd, F, routing=r)
        status_ok()
        close(out, ref.moe_experts(x, r.ids, r.wts, dgu, dd, F), 3e-2, 3e-2)


@pytest.mark.parametrize("nk,nv,dk,dv,tiled", [(2, 4, 128, 128, False), (2, 4, 128, 128, True), (2, 2, 64, 64, False),
                                                (1, 2, 64, 128, False)])
def test_gdn_prompt_kernel(nk, nv, dk, dv, tiled):
    """Prompt-sized chunks run the column-per-thread recurrence (one state column in registers per thread, token
    chunks staged by a producer warp): same outputs and final state as the fp32 reference, ragged lengths."""
    torch.manual_seed(dk + dv)
    lens = [70, 33, 9]
    cu = torch.tensor([0, 70, 103, 112], device=DEV, dtype=torch.int32)
    slots = torch.tensor([1, 3, 0], device=DEV, dtype=torch.int32)
    T = sum(lens)
    C = 2 * nk * dk + nv * dv
    x = rnd(T, C, scale=0.5)
    g = -torch.rand(T, nv, device=DEV) * 0.2
    beta = torch.rand(T, nv, device=DEV)
    st = torch.randn(4, nv, dk, dv, device=DEV) * 0.1
    st2 = st.clone()
    o = sm().gdn_recurrent(x, g, beta, st, cu, slots, nk, nv, dk, dv, tiled, dk ** -0.5)
    ro = ref.gdn_recurrent(x, g, beta, st2, cu, slots, nk, nv, dk, dv, tiled, dk ** -0.5)
    close(o, ro, 3e-2, 3e-2)
    close(st, st2, 2e-2, 2e-2)
    # verify rows: outputs without touching the state
    st3 = st2.clone()
    o2 = sm().gdn_recurrent(x, g, beta, st3, cu, slots, nk, nv, dk, dv, tiled, dk ** -0.5, write_state=False)
    assert torch.equal(st3, st2)
    assert o2.shape == o.shape


def _mla_reference(q_abs, cache, bt, ctx, cu, page, scale):
    """fp32 latent attention from the paged rows: softmax(q_abs . row) . row[:512], causal inside the step."""
    T, nh, _ = q_abs.shape
    out = torch.zeros(T, nh, 512, device=q_abs.device)
    rows = cache.reshape(-1, 576).float()
    for i in range(len(ctx)):
        q0, q1 = cu[i], cu[i + 1]
        c = ctx[i]
        nb = (c + page - 1) // page
        idx = (bt[i, :nb].long()[:, None] * page + torch.arange(page, device=q_abs.device)[None]).reshape(-1)[:c]
        lat = rows[idx]
        s = torch.einsum("qhd,kd->hqk", q_abs[q0:q1].float(), lat) * scale
        qpos = torch.arange(c - (q1 - q0), c, device=q_abs.device)[:, None]
        kpos = torch.arange(c, device=q_abs.device)[None]
        s = s.masked_fill((kpos > qpos)[None], float("-inf"))
        out[q0:q1] = torch.einsum("hqk,kl->qhl", torch.softmax(s, -1), lat[:, :512])
    return out


@pytest.mark.parametrize("nh,page,q_lens,ctx,splits", [
    (128, 64, [1, 1, 1], [70, 300, 1000], 1),       # decode, 2 head blocks per token
    (128, 16, [1, 1, 1], [70, 300, 1000], 3),       # split keys + combine, small pages
    (16, 64, [5, 1, 130], [5, 260, 200], 1),        # 4 tokens per tile: verify rows and a prompt chunk
    (64, 32, [3, 2], [515, 64], 2),
])
def test_mla_attn(nh, page, q_lens, ctx, splits):
    """tcgen05 latent attention (M = 64 tiles, S and O interleaved in TMEM) against the fp32 form."""
    torch.manual_seed(nh + page)
    n_blocks = 80
    cache = (torch.randn(n_blocks, page, 1, 576, device=DEV) * 0.5).bfloat16()
    width = (max(ctx) + page - 1) // page + 1
    bt = torch.stack([torch.randperm(n_blocks, device=DEV)[:width] for _ in q_lens]).int()
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    q_abs = (torch.randn(T, nh, 576, device=DEV) * 0.5).bfloat16()
    scale = 192 ** -0.5
    out = sm().mla_attn(q_abs, cache, torch.tensor(cu, device=DEV, dtype=torch.int32),
                        torch.tensor(ctx, device=DEV, dtype=torch.int32), bt, page, max(q_lens), scale,
                        n_splits=splits)
    status_ok()
    want = _mla_reference(q_abs, cache, bt, ctx, cu, page, scale)
    close(out, want, 3e-2, 3e-2)


def test_mla_prep():
    """Latent row norm + key rope + cache write + query rope in one launch against the reference ops."""
    torch.manual_seed(3)
    T, nh, dn = 7, 16, 32
    kva = rnd(T, 576)
    q = rnd(T, nh, dn + 64)
    nw = torch.rand(512, device=DEV) + 0.5
    cos_sin = ref.rope_cos_sin(256, 64, 10000.0, None, device=DEV)
    pos = torch.tensor([0, 5, 9, 100, 101, 255, 3], device=DEV, dtype=torch.int32)
    slots = torch.tensor([4, 130, -1, 17, 18, 0, 77], device=DEV, dtype=torch.int64)
    cache = torch.zeros(4, 64, 1, 576, device=DEV, dtype=torch.bfloat16)
    q_abs = torch.zeros(T, nh, 576, device=DEV, dtype=torch.bfloat16)
    sm().mla_prep(kva, nw, 1e-6, 0.0, q, dn, cos_sin, pos, slots, cache, q_abs)
    ckv, _ = ref.rmsnorm(kva[:, :512].contiguous(), nw, 1e-6, 0.0)
    kpe = ref.apply_rope(kva[:, 512:].reshape(T, 1, 64), cos_sin, pos, 64).reshape(T, 64)
    qpe = ref.apply_rope(q[..., dn:], cos_sin, pos, 64)
    rows = cache.view(-1, 576)
    for t in range(T):
        if slots[t] >= 0:
            close(rows[slots[t], :512], ckv[t], 2e-2, 2e-2)
            close(rows[slots[t], 512:], kpe[t], 2e-2, 2e-2)
    assert rows[2].abs().sum() == 0                       # the padding row wrote nothing
    close(q_abs[..., 512:], qpe, 2e-2, 2e-2)
    assert q_abs[..., :512].abs().sum() == 0


def _fp8_ref_linear(x, wq):
    """fp32 product of the de-quantised operands the FP8 GEMM sees (activations per row and 128 columns)."""
    x8, xs = sm().fp8_quant_act(x)
    xd = x8.view(torch.float8_e4m3fn).float() * xs.repeat_interleave(128, dim=1)
    d2, s2 = wq.view2d()
    wd = d2.view(torch.float8_e4m3fn).float() * \
        s2.repeat_interleave(128, dim=0)[:d2.shape[0]].repeat_interleave(128, dim=1)
    return xd, wd


@pytest.mark.parametrize("T,N,K", [(16, 5120, 2048), (1, 256, 128), (40, 384, 256), (100, 640, 1024), (33, 200, 384)])
def test_fp8_block_scaled_linear(T, N, K):
    """e4m3 weights with 128 x 128 block scales and e4m3 activations with 1 x 128 scales on the f8f6f4 tensor-core
    path, each 128-wide k block promoted into fp32 with its two scales (split-K included for the skinny shapes)."""
    torch.manual_seed(T + N)
    x = rnd(T, K)
    w = rnd(N, K, scale=0.05)
    res = rnd(T, N)
    wq = sm().Fp8Weight.quantize(w)
    out = sm().linear(x, wq, residual=res)
    status_ok()
    xd, wd = _fp8_ref_linear(x, wq)
    want = xd @ wd.t() + res.float()
    close(out, want, 1e-2, 1e-2)
    # and the quantisation itself stays near the bf16 product
    ref_full = x.float() @ w.float().t() + res.float()
    assert (out.float() - ref_full).abs().max() < 0.08 * ref_full.abs().max() + 0.05


def test_fp8_gate_up_and_experts():
    torch.manual_seed(11)
    T, H, F, E, k = 16, 512, 256, 8, 2
    x = rnd(T, H)
    wgu = rnd(2 * F, H, scale=0.05)
    q = sm().Fp8Weight.quantize(wgu)
    out = sm().gate_up_act(x, q, F)
    status_ok()
    xd, wd = _fp8_ref_linear(x, q)
    hh = xd @ wd.t()
    close(out, torch.nn.functional.silu(hh[:, :F]) * hh[:, F:], 2e-2, 2e-2)
    # routed experts: decode-sized step (dense routing tables) and a larger step (plan + gather)
    gu = rnd(E, 2 * F, H, scale=0.05)
    dn = rnd(E, H, F, scale=0.05)
    gq, dq = sm().Fp8Weight.quantize(gu), sm().Fp8Weight.quantize(dn)
    w_r = rnd(E, H, scale=0.1)
    for T2 in (16, 150):
        x2 = rnd(T2, H)
        routing = sm().router(x2, w_r, k)
        y = sm().moe_experts(x2, routing.ids, routing.wts, gq, dq, F, routing=routing)
        status_ok()
        want = ref.moe_experts(x2, routing.ids, routing.wts, gq.dequantize(), dq.dequantize(), F)
        err = (y.float() - want.float()).abs().max().item()
        assert err < 0.06 * want.abs().max().item() + 0.03, (T2, err)
        if T2 == 16:
            # the gate/up epilogue's own e4m3 encoding of the activated rows = the separate encoder's bytes
            sm().TUNE["fp8_fused_quant"] = 0
            try:
                y2 = sm().moe_experts(x2, routing.ids, routing.wts, gq, dq, F, routing=routing)
            finally:
                sm().TUNE["fp8_fused_quant"] = 1
            assert torch.equal(y, y2)


@pytest.mark.parametrize("T,nh,K,xcol,rpg,nf", [(16, 16, 128, 192, 512, 512), (70, 8, 512, 512, 256, 128),
                                                (300, 4, 64, 128, 128, 128)])
def test_head_linear_in_place_slices(T, nh, K, xcol, rpg, nf):
    """Per-head projections through one grouped GEMM launch: each head's activation slice is read in place (column
    offset in the TMA coordinate) and its output rows go through the row map."""
    torch.manual_seed(T)
    x = rnd(T, nh * xcol)
    w = rnd(nh * rpg, K, scale=0.1)
    ldo = nf + 64
    out = torch.zeros(T * nh, ldo, device=DEV, dtype=torch.bfloat16)
    sm().head_linear(x, w, nh, rpg, nf, K, xcol, out)
    status_ok()
    xs = x.view(T, nh, xcol)[:, :, :K].float()
    wh = w.view(nh, rpg, K)[:, :nf].float()
    want = torch.einsum("thk,hfk->thf", xs, wh).reshape(T * nh, nf)
    close(out[:, :nf], want, 2e-2, 2e-2)
    assert out[:, nf:].abs().sum() == 0


@pytest.mark.parametrize("nk,nv,d,tiled,n_seq", [(2, 4, 128, False, 5), (4, 8, 64, True, 16), (2, 2, 128, False, 1),
                                                (16, 32, 128, False, 3)])
def test_gdn_decode_fused_matches_the_separate_kernels(nk, nv, d, tiled, n_seq):
    """One launch (conv + gates + delta rule + gated norm) against the four-kernel path and the fp32 reference,
    outputs and both carried states, over two consecutive decode steps."""
    torch.manual_seed(nk * 7 + n_seq)
    C = 2 * nk * d + nv * d
    W = C + nv * d + 2 * nv
    conv_w = torch.randn(C, 4, device=DEV) * 0.5
    A = -torch.rand(nv, device=DEV) - 0.1
    dtb = torch.randn(nv, device=DEV)
    nw = torch.rand(d, device=DEV) + 0.5
    slots = torch.randperm(n_seq + 2, device=DEV)[:n_seq].int()
    cu = torch.arange(n_seq + 1, device=DEV, dtype=torch.int32)
    cst = [torch.randn(n_seq + 2, C, 3, device=DEV) for _ in range(3)]
    cst[1].copy_(cst[0]); cst[2].copy_(cst[0])
    sst = [torch.randn(n_seq + 2, nv, d, d, device=DEV) * 0.1 for _ in range(3)]
    sst[1].copy_(sst[0]); sst[2].copy_(sst[0])
    for step in range(2):
        proj = rnd(n_seq, W)
        out = sm().gdn_decode_fused(proj, conv_w, cst[0], A, dtb, nw, 1e-6, "silu", sst[0], slots, nk, nv, d, d, tiled,
                                    d ** -0.5)
        status_ok()
        mixed, z, ba = proj[:, :C], proj[:, C:C + nv * d], proj[:, C + nv * d:]
        outs = []
        for impl, k in ((sm(), 1), (ref, 2)):
            y = impl.causal_conv1d_silu(mixed, conv_w, None, cst[k], cu, slots)
            g, beta = impl.gdn_gates(ba[:, nv:], ba[:, :nv], A, dtb)
            o = impl.gdn_recurrent(y, g, beta, sst[k], cu, slots, nk, nv, d, d, tiled, d ** -0.5)
            zz = z if impl is not ref else z.reshape(n_seq, nv, d)
            outs.append(impl.gated_rmsnorm(o, zz, nw, 1e-6).reshape(n_seq, nv * d))
        close(out, outs[0], 1e-2, 1e-2)
        close(out, outs[1], 4e-2, 4e-2)
        close(cst[0], cst[1], 1e-6, 1e-6)
        close(sst[0][slots.long()], sst[1][slots.long()], 1e-3, 1e-3)
        close(sst[0][slots.long()], sst[2][slots.long()], 2e-2, 2e-2)


@pytest.mark.parametrize("nk,nv,tiled,lens", [(2, 4, False, [200]), (2, 2, True, [64, 130, 333]), (4, 8, False, [1000, 65]),
                                             (1, 2, False, [128])])
def test_gdn_chunked_scan_matches_token_serial(nk, nv, tiled, lens):
    """Chunked (64-token) tensor-core scan against the fp32 reference and the token-serial kernel: outputs of every
    token and the carried state, ragged lengths, non-zero initial state, a second step that continues from the
    written state."""
    torch.manual_seed(sum(lens) + nk)
    d = 128
    C = 2 * nk * d + nv * d
    n_seq = len(lens)
    slots = torch.randperm(n_seq + 1, device=DEV)[:n_seq].int()
    st = [torch.randn(n_seq + 1, nv, d, d, device=DEV) * 0.05 for _ in range(3)]
    st[1].copy_(st[0]); st[2].copy_(st[0])
    for step in range(2):
        T = sum(lens)
        cu_h = [0]
        for n in lens:
            cu_h.append(cu_h[-1] + n)
        cu = torch.tensor(cu_h, device=DEV, dtype=torch.int32)
        qkv = rnd(T, C, scale=0.5)
        g = -torch.rand(T, nv, device=DEV) * 0.15
        beta = torch.rand(T, nv, device=DEV)
        out = sm().gdn_chunked(qkv, g, beta, st[0], cu_h, slots, nk, nv, d, d, tiled, d ** -0.5)
        status_ok()
        want = ref.gdn_recurrent(qkv, g, beta, st[1], cu, slots, nk, nv, d, d, tiled, d ** -0.5)
        import legion_b200.ops.sm100 as S
        S.TUNE["gdn_chunk"] = 0
        try:
            serial = sm().gdn_recurrent(qkv, g, beta, st[2], cu, slots, nk, nv, d, d, tiled, d ** -0.5)
        finally:
            S.TUNE["gdn_chunk"] = 1
        scale = float(want.float().abs().max())
        assert float((out.float() - want.float()).abs().max()) < 0.03 * scale + 2e-3, "outputs vs reference"
        assert float((out.float() - serial.float()).abs().max()) < 0.03 * scale + 2e-3, "outputs vs token-serial kernel"
        sl = slots.long()
        ss = float(st[1][sl].abs().max())
        assert float((st[0][sl] - st[1][sl]).abs().max()) < 0.02 * ss + 2e-3, "state vs reference"
        lens = [max(1, n // 2 + 3) for n in lens]       # the next step continues every sequence


@pytest.mark.parametrize("lens", [[200], [70, 2, 1, 129], [64]])
def test_conv1d_token_parallel_form(lens):
    """Prompt-sized steps run the token-parallel convolution: outputs and carried history equal the reference,
    including sequences shorter than the kernel width."""
    torch.manual_seed(len(lens))
    C = 384
    T = sum(lens)
    cu_h = [0]
    for n in lens:
        cu_h.append(cu_h[-1] + n)
    cu = torch.tensor(cu_h, device=DEV, dtype=torch.int32)
    slots = torch.randperm(len(lens) + 1, device=DEV)[:len(lens)].int()
    x = rnd(T, C)
    w = torch.randn(C, 4, device=DEV) * 0.5
    cst = torch.randn(len(lens) + 1, C, 3, device=DEV)
    cst2 = cst.clone()
    y = sm().causal_conv1d_silu(x, w, None, cst, cu, slots, max_len=max(max(lens), 64))
    ry = ref.causal_conv1d_silu(x, w, None, cst2, cu, slots)
    close(y, ry)
    close(cst, cst2, 1e-5, 1e-5)


@pytest.mark.parametrize("nh,hd,ng,ds,lens", [(8, 64, 1, 128, [1, 1, 1]), (8, 32, 2, 32, [37, 1, 130]), (4, 128, 4, 64, [300])])
def test_mamba2_scan_matches_token_serial_reference(nh, hd, ng, ds, lens):
    """State-space recurrence + D skip + silu(z) gate against the fp32 token loop; decode rows, ragged prompts, a
    chunk that continues from a carried state."""
    from legion_b200.ops import sm100
    torch.manual_seed(1)
    dev = "cuda"
    di, T, n = nh * hd, sum(lens), len(lens)
    xbc = (torch.randn(T, di + 2 * ng * ds, device=dev) * 0.5).bfloat16()
    dt = torch.randn(T, nh, device=dev).bfloat16()
    z = torch.randn(T, di, device=dev).bfloat16()
    A = -torch.rand(nh, device=dev) - 0.1
    D = torch.randn(nh, device=dev)
    dtb = torch.randn(nh, device=dev) * 0.3
    state = torch.randn(n + 2, nh, hd, ds, device=dev) * 0.2
    slots = torch.tensor([n + 1 - i for i in range(n)], dtype=torch.int32, device=dev)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    want_state = state.clone()
    want = torch.empty(T, di, device=dev)
    hg = nh // ng
    for i in range(n):
        S = want_state[int(slots[i])].clone()
        for t in range(int(cu[i]), int(cu[i + 1])):
            dtv = torch.nn.functional.softplus(dt[t].float() + dtb)
            xs = xbc[t, :di].float().view(nh, hd)
            Bt = xbc[t, di:di + ng * ds].float().view(ng, ds).repeat_interleave(hg, 0)
            Ct = xbc[t, di + ng * ds:].float().view(ng, ds).repeat_interleave(hg, 0)
            S = S * torch.exp(dtv * A)[:, None, None] + (dtv[:, None] * xs)[:, :, None] * Bt[:, None, :]
            yv = torch.einsum("hds,hs->hd", S, Ct) + D[:, None] * xs
            want[t] = (yv.reshape(di) * torch.nn.functional.silu(z[t].float()))
        want_state[int(slots[i])] = S
    keep = state.clone()
    got = sm100.mamba2_scan(xbc, dt, z, A, D, dtb, state, cu, slots, nh, hd, ng, ds, write_state=False)
    assert torch.equal(state, keep)                       # verify rows leave the state alone
    got = sm100.mamba2_scan(xbc, dt, z, A, D, dtb, state, cu, slots, nh, hd, ng, ds)
    assert float((got.float() - want).abs().max()) < 0.02 * float(want.abs().max()) + 0.02
    assert float((state - want_state).abs().max()) < 1e-3 * float(want_state.abs().max()) + 1e-4


# ------------------------------------------------------------------------------------------------
# long contexts: the same kernels at 8K and 32K keys (block tables of hundreds of pages, many key
# splits, accumulation over hundreds of tiles)
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("D,Hq,Hkv,page,ctx", [(128, 32, 4, 64, [8192, 32768, 5001]), (256, 16, 2, 64, [32768, 8193]),
                                               (128, 8, 8, 16, [8192, 1, 12000])])
def test_paged_decode_long_context(D, Hq, Hkv, page, ctx):
    torch.manual_seed(D + Hq + page)
    B = len(ctx)
    width = (max(ctx) + page - 1) // page
    n_blocks = width + 40
    kc, vc = make_cache(n_blocks, page, Hkv, D)
    bt = torch.stack([torch.randperm(n_blocks, device=DEV)[:width] for _ in range(B)]).int()
    q = rnd(B, Hq, D)
    ctx_t = torch.tensor(ctx, device=DEV, dtype=torch.int32)
    scale = D ** -0.5
    want = ref.paged_attention(q, kc, vc, bt, ctx_t, torch.arange(B + 1), scale)
    for ns in (None, 1, 7):
        out = sm().paged_decode(q, kc, vc, bt, ctx_t, scale, n_splits=ns)
        status_ok()
        close(out, want, 2e-2, 2e-2)
    wantw = ref.paged_attention(q, kc, vc, bt, ctx_t, torch.arange(B + 1), scale, window=4096)
    close(sm().paged_decode(q, kc, vc, bt, ctx_t, scale, window=4096), wantw, 2e-2, 2e-2)
    status_ok()


@pytest.mark.parametrize("D,Hq,Hkv,page,q_lens,ctx", [(128, 4, 2, 64, [1024, 300], [32768, 8192 + 300]),
                                                      (256, 2, 1, 64, [700], [8192 + 700]),
                                                      (128, 4, 4, 32, [8192], [8192])])
def test_prefill_attn_long_context(D, Hq, Hkv, page, q_lens, ctx):
    """Prompt chunks at the end of 8K / 32K keys already in the cache, and one whole 8K prompt."""
    torch.manual_seed(D + page + len(q_lens))
    width = (max(ctx) + page - 1) // page + 1
    n_blocks = width + 30
    kc, vc = make_cache(n_blocks, page, Hkv, D)
    bt = torch.stack([torch.randperm(n_blocks, device=DEV)[:width] for _ in q_lens]).int()
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    cu_t = torch.tensor(cu, device=DEV, dtype=torch.int32)
    q = rnd(cu[-1], Hq, D)
    ctx_t = torch.tensor(ctx, device=DEV, dtype=torch.int32)
    scale = D ** -0.5
    out = sm().prefill_attn(q, kc, vc, cu_t, ctx_t, bt, max(q_lens), scale)
    status_ok()
    want = ref.paged_attention(q, kc, vc, bt, ctx_t, cu_t, scale)
    close(out, want, 3e-2, 3e-2)


@pytest.mark.parametrize("nh,page,q_lens,ctx,splits", [(128, 64, [1, 1], [8192, 32768], None),
                                                       (16, 64, [130, 1], [8192 + 130, 20000], 5)])
def test_mla_attn_long_context(nh, page, q_lens, ctx, splits):
    torch.manual_seed(nh + len(ctx))
    width = (max(ctx) + page - 1) // page + 1
    n_blocks = width + 20
    cache = (torch.randn(n_blocks, page, 1, 576, device=DEV) * 0.5).bfloat16()
    bt = torch.stack([torch.randperm(n_blocks, device=DEV)[:width] for _ in q_lens]).int()
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    q_abs = (torch.randn(cu[-1], nh, 576, device=DEV) * 0.5).bfloat16()
    scale = 192 ** -0.5
    out = sm().mla_attn(q_abs, cache, torch.tensor(cu, device=DEV, dtype=torch.int32),
                        torch.tensor(ctx, device=DEV, dtype=torch.int32), bt, page, max(q_lens), scale, n_splits=splits)
    status_ok()
    close(out, _mla_reference(q_abs, cache, bt, ctx, cu, page, scale), 3e-2, 3e-2)


def test_scratch_buffers_keep_their_guard_areas(monkeypatch):
    """Debug build of the scratch allocator (``LB_CANARY=1``): every cached scratch tensor sits between two guard
    areas; after a decode-sized MoE block, a router call on wide rows, an arg-max and a split-key attention call none
    of the guards has been written."""
    import legion_b200.ops.sm100 as m
    monkeypatch.setattr(m, "_CANARY_ON", True)
    saved = dict(m.Workspace._by_device)
    m.Workspace._by_device.clear()
    try:
        T, E, k, H, F = 16, 32, 4, 4096, 256
        x, res = rnd(T, H), rnd(T, H)
        nw = torch.rand(H, device=DEV) + 0.5
        r = m.router(x, rnd(E, H, scale=H ** -0.5), k, norm=(nw, 1e-6, 0.0))
        m.moe_experts(r.x_normed, r.ids, r.wts, rnd(E, 2 * F, H, scale=H ** -0.5), rnd(E, H, F, scale=F ** -0.5), F,
                      residual=res, routing=r)
        m.argmax(torch.randn(5, 70000, device=DEV))
        Hq, Hkv, D, page, ctx = 8, 2, 128, 64, 700
        nb = 3 * ((ctx + page - 1) // page)
        kc, vc = make_cache(nb, page, Hkv, D)
        bt = torch.arange(nb, device=DEV, dtype=torch.int32).view(3, -1)
        m.paged_decode(rnd(3, Hq, D), kc, vc, bt, torch.full((3,), ctx, device=DEV, dtype=torch.int32), D ** -0.5,
                       n_splits=4, max_ctx=ctx)
        ws = m.Workspace.get(DEV)
        assert len(ws._guards) >= 3
        assert ws.check() == 0 and ws.check_canaries() == []
        # the check itself: a byte written just past a buffer is reported under the buffer's name
        key, raw = next(iter(ws._guards.items()))
        raw[-1] = 0
        assert ws.check_canaries() == [str(key[0])]
    finally:
        m.Workspace._by_device.clear()
        m.Workspace._by_device.update(saved)
