"""``comm-bench``: device-timed micro-benchmarks of the fused communication kernels against their NCCL forms.

Run one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m legion_b200.bench.comm --hidden 2048 --rows 16,64,2048 --json out.json

Every row of the table is a CUDA graph of ``--iters`` calls, replayed ``--reps`` times between two CUDA events
(median), max over ranks; a grid-wide barrier precedes every replay. Columns:

  * ``fused_us`` ......... one-shot (decode sizes) or two-shot (prompt sizes) all-reduce + residual + RMSNorm in the
                           symmetric-memory kernels; ``fused_q_us`` with the NVFP4 encoding of the normalised rows
                           out of the same launch.
  * ``nccl_us`` .......... ``dist.all_reduce`` + the residual-add + RMSNorm kernel (the baseline path).
  * ``gemm_ar_us`` ....... projection GEMM + reduction in ONE kernel (``linear_reduce_norm``) against
                           ``gemm_then_ar_us`` = the GEMM writing into the slot followed by the reduction kernel.
  * ``ag_gemm_us`` ....... all-gather + GEMM in one kernel (``all_gather_linear``) against ``nccl_ag_gemm_us``.
  * ``link_frac`` ........ bytes that must cross NVLink per GPU and direction (one-shot: (W - 1) x rows x H x 2
                           loaded from the peers) divided by time x 770 GB/s, the measured peer-copy bandwidth.

Reference counterpart: the all-reduce figures of ``docs/bench.md`` (their TP latency table) and
``src/tp_net/op.rs:26-60``.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys

PEER_GBS = 770.0


def _graph_time(fn, iters: int, reps: int, dev) -> float:
    """Median µs per call of ``fn`` inside a replayed graph of ``iters`` calls (max over ranks)."""
    import torch
    import torch.distributed as dist
    s = torch.cuda.Stream(device=dev)
    s.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(s):
        for _ in range(2):
            fn()
    torch.cuda.current_stream(dev).wait_stream(s)
    torch.cuda.synchronize(dev)
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(iters):
            fn()
    times = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(reps + 2):
        dist.barrier()
        torch.cuda.synchronize(dev)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize(dev)
        times.append(e0.elapsed_time(e1) * 1e3 / iters)
    t = torch.tensor([statistics.median(times[2:])], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="comm-bench")
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--rows", default="16,64,2048")
    ap.add_argument("--proj-k", type=int, default=0, help="K of the projection in the GEMM rows (0 = hidden / world * 2)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--reps", type=int, default=7)
    ap.add_argument("--json")
    a = ap.parse_args(argv)

    import torch
    import torch.distributed as dist

    from ..ops import sm100
    from . import kernels as _k  # noqa: F401  (same extension)
    from ..parallel import dist as pdist

    rank, local_rank, world = pdist.env_world()
    if world < 2:
        print("comm-bench needs at least two ranks (torch.distributed.run --nproc-per-node N)", file=sys.stderr)
        return 2
    H = a.hidden
    rows = [int(r) for r in a.rows.split(",") if r.strip()]
    pctx = pdist.init_from_env("cuda", comm="fused", max_rows=max(rows), hidden=H)
    dev = torch.device("cuda", local_rank)
    comm = pctx.symm
    torch.manual_seed(3 + rank)
    w_norm = torch.rand(H, device=dev) + 0.5
    out = {"world": world, "hidden": H, "peer_gbs": PEER_GBS, "rows": []}
    for T in rows:
        res = torch.randn(T, H, device=dev).bfloat16()
        part = (torch.randn(T, H, device=dev) * 0.5).bfloat16()
        K = a.proj_k or max(256, 2 * H // world)
        x = (torch.randn(T, K, device=dev) * 0.3).bfloat16()
        wp = (torch.randn(H, K, device=dev) * 0.05).bfloat16()
        row = {"rows": T}

        def fused(quant=False):
            for _ in range(2):      # an even number of reductions keeps the slot rotation of a step
                slot = comm.next_partial(T, H)
                comm.all_reduce_add_norm(slot, res, w_norm, 1e-6, 0.0, quant=quant)

        for _ in range(2):
            comm.next_partial(T, H).copy_(part)
            comm._advance()
        row["fused_us"] = _graph_time(fused, a.iters, a.reps, dev) / 2
        if T <= 64 and H % 256 == 0:
            row["fused_q_us"] = _graph_time(lambda: fused(True), a.iters, a.reps, dev) / 2

        buf = part.clone()

        def nccl():
            dist.all_reduce(buf)
            sm100.rmsnorm(buf, w_norm, 1e-6, 0.0, res)

        row["nccl_us"] = _graph_time(nccl, a.iters, a.reps, dev)

        def gemm_then_ar():
            for _ in range(2):
                slot = comm.next_partial(T, H)
                sm100.linear(x, wp, out=slot)
                comm.all_reduce_add_norm(slot, res, w_norm, 1e-6, 0.0)

        row["gemm_then_ar_us"] = _graph_time(gemm_then_ar, a.iters, a.reps, dev) / 2
        if comm.fits_gemm_tail(T, H):
            def gemm_ar():
                for _ in range(2):
                    comm.linear_reduce_norm(x, wp, res, w_norm, 1e-6, 0.0)
            row["gemm_ar_us"] = _graph_time(gemm_ar, a.iters, a.reps, dev) / 2

        # all-gather -> GEMM (sequence-parallel layout: every rank holds rows / world of the activation)
        wq = (torch.randn(2 * H, H, device=dev) * 0.05).bfloat16()
        r0, n, _ = comm.shard_rows(T)
        xs = (torch.randn(T, H, device=dev) * 0.3).bfloat16()

        def ag_gemm():
            for _ in range(2):
                comm.shard_view(T).copy_(xs[r0:r0 + n])
                comm.all_gather_linear(T, wq)

        row["ag_gemm_us"] = _graph_time(ag_gemm, a.iters, a.reps, dev) / 2
        per = (T + world - 1) // world
        xa = torch.empty(per * world, H, dtype=torch.bfloat16, device=dev)
        xpad = torch.zeros(per, H, dtype=torch.bfloat16, device=dev)
        xpad[:n] = xs[r0:r0 + n]

        def nccl_ag_gemm():
            dist.all_gather_into_tensor(xa, xpad)
            sm100.linear(xa[:T], wq)

        row["nccl_ag_gemm_us"] = _graph_time(nccl_ag_gemm, a.iters, a.reps, dev)
        one_shot = not (T >= comm.TWO_SHOT_ROWS and world > 2)
        link_bytes = (world - 1) * T * H * 2 if one_shot else 2 * (world - 1) * T * H * 2 / world
        row["link_bytes"] = int(link_bytes)
        row["link_frac"] = round(link_bytes / (row["fused_us"] * 1e-6) / (PEER_GBS * 1e9), 4)
        row["ag_link_frac"] = round((world - 1) * per * H * 2 / (row["ag_gemm_us"] * 1e-6) / (PEER_GBS * 1e9), 4)
        gemm_flops = 2.0 * T * (2 * H) * H
        row["ag_gemm_tflops"] = round(gemm_flops / (row["ag_gemm_us"] * 1e-6) / 1e12, 2)
        out["rows"].append({k: (round(v, 2) if isinstance(v, float) else v) for k, v in row.items()})
        comm.check()
    assert sm100.Workspace.get(dev).check() == 0
    if rank == 0:
        for r in out["rows"]:
            print(json.dumps(r))
        if a.json:
            with open(a.json, "w") as f:
                json.dump(out, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
