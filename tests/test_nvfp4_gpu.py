"""Native NVFP4 (W4A4) path: scale-atom layout, activation quantiser (plain and fused with RMSNorm), and the
block-scaled tcgen05 GEMM in its dense, gate/up (+ SwiGLU), grouped and quantised-output forms, each against the
fp32 product of the de-quantised operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda")


def _w(rows, K, seed, std=0.05):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(rows, K, generator=g) * std).bfloat16().to(_dev())


def test_scale_atoms_round_trip():
    from legion_b200.ops import sm100
    C = sm100.ext()
    for rows, K in ((128, 256), (300, 2048), (512, 192)):
        lin = torch.randint(1, 127, (rows, K // 16), dtype=torch.uint8, device=_dev())
        atoms = torch.zeros(C.nv4_sf_bytes(rows, K), dtype=torch.uint8, device=_dev())
        C.nv4_pack_scales(lin, atoms)
        back = torch.zeros_like(lin)
        C.nv4_unpack_scales(atoms, back)
        assert torch.equal(back, lin)
        # spot check of the documented position: row r, block b
        r, b = rows - 3, K // 16 - 1
        k4 = ((K + 255) // 256) * 4
        off = ((r >> 7) * k4 + (b >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (b & 3)
        assert int(atoms[off]) == int(lin[r, b])


def test_activation_quantiser_plain_and_with_rmsnorm():
    from legion_b200.ops import reference as ref
    from legion_b200.ops import sm100
    torch.manual_seed(0)
    for T, K in ((5, 2048), (40, 512), (130, 4096)):
        x = (torch.randn(T, K, device=_dev()) * torch.rand(T, 1, device=_dev()) * 3).bfloat16()
        q = sm100.nv4_quant_act(x)
        deq = q.dequantize()
        blk = x.float().view(T, K // 16, 16).abs().amax(-1, keepdim=True).expand(T, K // 16, 16).reshape(T, K)
        err = (deq - x.float()).abs()
        assert float((err - 0.19 * blk).max()) <= 1e-6          # half of the coarsest e2m1 step (+ scale rounding)
        assert float(err.mean() / x.float().abs().mean()) < 0.12
        # fused residual add + RMSNorm + quantisation
        res = torch.randn(T, K, device=_dev()).bfloat16()
        w = torch.rand(K, device=_dev()) + 0.5
        q2 = sm100.nv4_quant_act(x, norm=(w, 1e-6, 0.0), residual=res, want_normed=True)
        summed = (x.float() + res.float()).bfloat16()
        want_n, _ = ref.rmsnorm(summed, w, 1e-6)
        assert torch.equal(q2.summed, summed)
        assert float((q2.normed.float() - want_n.float()).abs().max()) < 0.04
        q3 = sm100.nv4_quant_act(q2.normed)
        assert torch.equal(q3.codes, q2.codes) and torch.equal(q3.gscale[:T], q2.gscale[:T])


@pytest.mark.parametrize("T,N,K,bn", [(16, 256, 2048, 32), (50, 384, 512, 64), (1, 128, 256, 32), (200, 512, 1024, 128),
                                      (33, 256, 320, 64)])
def test_dense_linear_matches_dequantised_product(T, N, K, bn):
    from legion_b200.ops import sm100
    w = _w(N, K, 1)
    x = (torch.randn(T, K, device=_dev()) * 0.7).bfloat16()
    qw = sm100.Nv4Weight.quantize_cuda(w)
    qx = sm100.nv4_quant_act(x)
    res = torch.randn(T, N, device=_dev()).bfloat16()
    out = sm100.linear_nv4(qx, qw, residual=res, bn=bn)
    want = qx.dequantize() @ qw.dequantize(torch.float32).t() + res.float()
    assert sm100.Workspace.get(_dev()).check() == 0
    assert float((out.float() - want).abs().max()) < 0.02 * float(want.abs().max()) + 1e-3
    # the quantised product itself is close to the bf16 one (4-bit noise)
    full = x.float() @ w.float().t() + res.float()
    assert float((out.float() - full).abs().mean() / full.abs().mean()) < 0.2


@pytest.mark.parametrize("T,F,K,bn", [(16, 512, 2048, 32), (64, 256, 512, 64)])
def test_gate_up_swiglu_bf16_and_quantised_output(T, F, K, bn):
    from legion_b200.ops import sm100
    w = _w(2 * F, K, 2)
    x = (torch.randn(T, K, device=_dev()) * 0.7).bfloat16()
    qw = sm100.Nv4Weight.quantize_cuda(w, dual_rows=F)
    qx = sm100.nv4_quant_act(x)
    h = sm100.gate_up_nv4(qx, qw, F, bn=bn)
    wd = qw.dequantize(torch.float32)
    xd = qx.dequantize()
    g, u = xd @ wd[:F].t(), xd @ wd[F:].t()
    want = torch.nn.functional.silu(g) * u
    assert float((h.float() - want).abs().max()) < 0.02 * float(want.abs().max()) + 1e-3
    # re-encoded output: de-quantising it gives the SwiGLU result up to 4-bit rounding, and a down projection from
    # it equals the product of the de-quantised operands
    qs = torch.tensor([float(want.abs().max()) / (6 * 448)], device=_dev())
    hq = sm100.gate_up_nv4(qx, qw, F, bn=bn, q_scale=qs)
    hd = hq.dequantize()
    blk = want.view(T, F // 16, 16).abs().amax(-1, keepdim=True).expand(T, F // 16, 16).reshape(T, F)
    assert float(((hd - want).abs() - 0.2 * blk).max()) <= 2e-3
    wdn = sm100.Nv4Weight.quantize_cuda(_w(256, F, 3))
    y = sm100.linear_nv4(hq, wdn)
    want_y = hd @ wdn.dequantize(torch.float32).t()
    assert sm100.Workspace.get(_dev()).check() == 0
    assert float((y.float() - want_y).abs().max()) < 0.02 * float(want_y.abs().max()) + 1e-3


def _moe_setup(T, E, k, H, F, seed):
    torch.manual_seed(seed)
    dev = _dev()
    x = (torch.randn(T, H, device=dev) * 0.8).bfloat16()
    res = torch.randn(T, H, device=dev).bfloat16()
    w_r = (torch.randn(E, H, device=dev) * H ** -0.5).bfloat16()
    wgu = (torch.randn(E + 1, 2 * F, H, device=dev) * H ** -0.5).bfloat16()      # last group = shared expert
    wd = (torch.randn(E + 1, H, F, device=dev) * F ** -0.5).bfloat16()
    sh_gate = (torch.randn(1, H, device=dev) * H ** -0.5).bfloat16()
    return x, res, w_r, wgu, wd, sh_gate


def _moe_reference(x, ids, wts, wgu, wd, F, sh_gate, res, E):
    from legion_b200.ops import reference as ref
    y = ref.moe_experts(x, ids, wts, wgu[:E], wd[:E], F)
    hs = ref.gate_up_act(x, wgu[E], F, "silu")
    sh = ref.linear(hs, wd[E]).float()
    gate = torch.sigmoid(ref.linear(x, sh_gate, out_dtype=torch.float32).reshape(-1))
    return y.float() + sh * gate[:, None] + res.float()


@pytest.mark.parametrize("T,E,k,H,F", [(16, 64, 4, 512, 256), (1, 16, 2, 256, 128), (40, 32, 6, 512, 256)])
def test_shared_expert_as_a_slot_of_the_grouped_gemms_bf16(T, E, k, H, F):
    """The shared expert stacked behind the routed experts runs as one more slot of the dense routing; its sigmoid
    gate comes out of the routing launch."""
    from legion_b200.ops import sm100
    x, res, w_r, wgu, wd, sh_gate = _moe_setup(T, E, k, H, F, 5)
    r = sm100.router(x, w_r, k, shared_slot=True, sh_gate=sh_gate)
    assert r.shared_slot and r.dense is not None
    out = sm100.moe_experts(x, r.ids, r.wts, wgu, wd, F, residual=res, routing=r)
    assert sm100.Workspace.get(_dev()).check() == 0
    want = _moe_reference(x, r.ids, r.wts, wgu, wd, F, sh_gate, res, E)
    assert float((out.float() - want).abs().max()) < 0.03 * float(want.abs().max()) + 0.03
    n_act = int(torch.unique(r.ids).numel())
    assert r.dense.meta.tolist() == [n_act + 1, (n_act + 1) * r.dense.stride]


@pytest.mark.parametrize("T,E,k,H,F", [(16, 64, 4, 512, 256), (3, 16, 2, 256, 256), (48, 32, 6, 1024, 512)])
def test_moe_block_native_nvfp4_with_shared_slot(T, E, k, H, F):
    """Routed + shared experts on the W4A4 path: quantised input, gate/up with re-encoded SwiGLU output, down,
    combine; against the fp32 computation over the de-quantised weights and activations."""
    from legion_b200.ops import reference as ref
    from legion_b200.ops import sm100
    x, res, w_r, wgu, wd, sh_gate = _moe_setup(T, E, k, H, F, 9)
    qgu = sm100.Nv4Weight.quantize_cuda(wgu, dual_rows=F)
    qdn = sm100.Nv4Weight.quantize_cuda(wd)
    r = sm100.router(x, w_r, k, shared_slot=True, sh_gate=sh_gate, slot_stride=128)
    out = sm100.moe_experts(x, r.ids, r.wts, qgu, qdn, F, residual=res, routing=r)
    assert sm100.Workspace.get(_dev()).check() == 0
    # reference: same quantised operands, intermediate re-encoded with the same static scale
    xd = sm100.nv4_quant_act(x).dequantize().bfloat16()
    gud, dnd = qgu.dequantize(torch.float32), qdn.dequantize(torch.float32)
    want_exact = _moe_reference(xd, r.ids, r.wts, gud.bfloat16(), dnd.bfloat16(), F, sh_gate, res, E)
    rel = float((out.float() - want_exact).abs().mean() / want_exact.abs().mean())
    assert rel < 0.08, rel                      # 4-bit rounding of the intermediate is the only difference
    full = _moe_reference(x, r.ids, r.wts, wgu, wd, F, sh_gate, res, E)
    assert float((out.float() - full).abs().mean() / full.abs().mean()) < 0.2
    out2 = sm100.moe_experts(x, r.ids, r.wts, qgu, qdn, F, residual=res, routing=r)
    assert torch.equal(out, out2)
    # a prompt-sized step with the same weights takes the plan path (de-quantising GEMM), routed experts only
    T2 = 200
    x2 = (torch.randn(T2, H, device=_dev()) * 0.8).bfloat16()
    r2 = sm100.router(x2, w_r, k)
    y2 = sm100.moe_experts(x2, r2.ids, r2.wts, qgu.narrow(0, E), qdn.narrow(0, E), F)
    want2 = ref.moe_experts(x2, r2.ids, r2.wts, gud[:E].bfloat16(), dnd[:E].bfloat16(), F)
    assert sm100.Workspace.get(_dev()).check() == 0
    assert float((y2.float() - want2.float()).abs().max()) < 0.03 * float(want2.abs().max()) + 0.03


@pytest.mark.parametrize("T,E,k,H,F,bn", [(1500, 32, 6, 512, 256, 64), (700, 16, 4, 1024, 512, 64),
                                          (2100, 24, 3, 512, 512, 128),
                                          (4000, 32, 8, 512, 256, 64)])     # >= 256 tiles: two epilogue warpgroups
def test_moe_block_native_nvfp4_prompt_sized(T, E, k, H, F, bn):
    """Prompt-sized steps: aligned routing plan, gather of the encoded rows, both grouped GEMMs on the W4A4 path.
    Against the fp32 computation over the de-quantised weights and activations."""
    from legion_b200.ops import reference as ref
    from legion_b200.ops import sm100
    x, res, w_r, wgu, wd, _ = _moe_setup(T, E, k, H, F, 11)
    qgu = sm100.Nv4Weight.quantize_cuda(wgu[:E].contiguous(), dual_rows=F)
    qdn = sm100.Nv4Weight.quantize_cuda(wd[:E].contiguous())
    r = sm100.router(x, w_r, k)
    # one expert gets no token at all: its segment is empty
    ids = torch.where(r.ids == 3, torch.full_like(r.ids, 5), r.ids)
    old = sm100.TUNE["nv4_sorted_bn"]
    sm100.TUNE["nv4_sorted_bn"] = bn
    try:
        out = sm100._moe_experts_nv4_sorted(x, ids, r.wts, qgu, qdn, F, 0, None, None, res, None, None)
        out2 = sm100._moe_experts_nv4_sorted(x, ids, r.wts, qgu, qdn, F, 0, None, None, res, None, None)
    finally:
        sm100.TUNE["nv4_sorted_bn"] = old
    assert sm100.Workspace.get(_dev()).check() == 0
    assert torch.equal(out, out2)                 # the order inside a segment does not reach the result
    xd = sm100.nv4_quant_act(x).dequantize().bfloat16()
    gud, dnd = qgu.dequantize(torch.float32), qdn.dequantize(torch.float32)
    want = ref.moe_experts(xd, ids, r.wts, gud.bfloat16(), dnd.bfloat16(), F).float() + res.float()
    rel = float((out.float() - want).abs().mean() / want.abs().mean())
    assert rel < 0.08, rel
    # the plan itself: segments on tile boundaries, every pair exactly once, padding rows marked
    plan = next(v for kk, v in sm100.Workspace.get(_dev())._cache.items()
                if isinstance(kk, tuple) and kk[0] == "nv4_plan" and kk[1] >= T and kk[1] < 2 * max(T, 1024)
                and kk[2] == k and kk[3] == E and kk[4] == bn and kk[5] == H and kk[6] == F)
    off = plan.offsets[:E + 1].tolist()
    cnt = torch.bincount(ids.reshape(-1).long(), minlength=E).tolist()
    assert all(o % bn == 0 for o in off) and cnt[3] == 0 and off[4] == off[3]
    st, sp = plan.sorted_token.cpu(), plan.sorted_pair.cpu()
    for e in range(E):
        seg = sp[off[e]:off[e] + cnt[e]].long()
        assert bool((ids.reshape(-1).cpu()[seg] == e).all()) and seg.unique().numel() == cnt[e]
        assert bool((st[off[e] + cnt[e]:off[e + 1]] == -1).all())
    assert plan.meta.tolist()[0] == sum((c + bn - 1) // bn for c in cnt)
