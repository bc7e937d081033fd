"""One MoE block of the 80B-A3B expert shape at decode size on the native NVFP4 path, run a few times: the small,
fixed case that the profiler captures are taken on (``ncu -k regex:<kernel> ... python -m
legion_b200.bench.moe_block_case``). Prints the status word."""
import sys

import torch


def main(argv=None):
    from legion_b200.ops import sm100
    from legion_b200.ops.sm100 import Nv4Weight
    T = int(argv[0]) if argv else 16
    H, E, k, F = 2048, 512, 10, 512
    dev = "cuda"
    C = sm100.ext()
    G = E + 1
    torch.manual_seed(0)
    x = torch.randn(T, H, device=dev).bfloat16()
    res = torch.randn(T, H, device=dev).bfloat16()
    nw = torch.ones(H, device=dev)
    w_r = (torch.randn(E, H, device=dev) * 0.02).bfloat16()
    sh_gate = (torch.randn(1, H, device=dev) * 0.02).bfloat16()

    def rand_w(rows, K):
        codes = torch.randint(0, 256, (G, rows, K // 2), device=dev, dtype=torch.uint8)
        lin = torch.randint(48, 64, (G * rows, K // 16), device=dev, dtype=torch.uint8)
        atoms = torch.zeros(C.nv4_sf_bytes(G * rows, K), dtype=torch.uint8, device=dev)
        C.nv4_pack_scales(lin, atoms)
        return codes, atoms
    gc, gs = rand_w(2 * F, H)
    dc, ds = rand_w(H, F)
    qgu = Nv4Weight(gc, gs, torch.full((2 * G,), 1e-3, device=dev))
    qdn = Nv4Weight(dc, ds, torch.full((G,), 1e-3, device=dev))
    flush = torch.zeros(64 << 20, dtype=torch.int32, device=dev)
    for _ in range(4):
        flush.sum()
        xq = sm100.nv4_quant_act(x, norm=(nw, 1e-6, 0.0), residual=res, want_normed=True, key="case_x")
        r = sm100.router(xq.normed, w_r, k, shared_slot=True, sh_gate=sh_gate, slot_stride=128)
        sm100._moe_experts_nv4(xq.normed, r.ids, r.wts, qgu, qdn, F, 0, None, None, xq.summed, None, (nw, 1e-6, 0.0), r,
                               xq=xq)
    torch.cuda.synchronize()
    print("status word:", sm100.Workspace.get(dev).check())


if __name__ == "__main__":
    main(sys.argv[1:])
