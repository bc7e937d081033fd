"""Fused collectives over symmetric memory on 2+ GPUs (child processes, one per GPU): the all-reduce + residual +
RMSNorm kernel, the two-shot form, a GEMM whose epilogue writes into the symmetric slot, and a TP engine."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _init(rank, world, port):
    import datetime
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=120), device_id=torch.device("cuda", rank))
    return dist


def _comm_worker(rank, world, port, out_path):
    dist = _init(rank, world, port)
    from legion_b200.ops import reference as ref
    from legion_b200.ops import sm100
    from legion_b200.parallel.symm import SymmComm
    dev = torch.device("cuda", rank)
    H = 512
    comm = SymmComm(dist.group.WORLD, rank, world, dev, max_rows=2048, hidden=H)
    torch.manual_seed(7)
    errs = []
    for T in (1, 16, 600, 2048):           # one-shot sizes and (world > 2) two-shot sizes
        parts = [(torch.randn(T, H, device=dev) * 0.5).bfloat16() for _ in range(world)]     # same on every rank
        res = torch.randn(T, H, device=dev).bfloat16()
        w = torch.rand(H, device=dev) + 0.5
        slot = comm.next_partial(T, H)
        slot.copy_(parts[rank])
        normed, summed = comm.all_reduce_add_norm(slot, res, w, 1e-6, 0.0)
        total = sum(p.float() for p in parts) + res.float()
        want_n, _ = ref.rmsnorm(total.bfloat16(), w, 1e-6)
        errs.append(float((summed.float() - total).abs().max()))
        errs.append(float((normed.float() - want_n.float()).abs().max()))
        # every rank must hold the same bits (rank-order sums)
        gathered = [torch.empty_like(summed) for _ in range(world)]
        dist.all_gather(gathered, summed)
        assert all(torch.equal(g, gathered[0]) for g in gathered)
    # GEMM epilogue writes straight into the slot, then the fused reduction
    x = (torch.randn(24, 256, device=dev) * 0.3).bfloat16()
    wts = [(torch.randn(H, 256, device=dev) * 0.05).bfloat16() for _ in range(world)]
    res = torch.randn(24, H, device=dev).bfloat16()
    slot = comm.next_partial(24, H)
    sm100.linear(x, wts[rank], out=slot)
    assert comm.owns(slot)
    _, summed = comm.all_reduce_add_norm(slot, res, None, 0.0, 0.0)
    want = sum(ref.linear(x, wt).float() for wt in wts) + res.float()
    errs.append(float((summed.float() - want).abs().max()))
    comm.end_step()
    comm.check()
    torch.cuda.synchronize()
    assert sm100.Workspace.get(dev).check() == 0
    if rank == 0:
        torch.save(errs, out_path)
    dist.barrier()
    dist.destroy_process_group()


def _engine_worker(rank, world, port, comm_kind, out_path):
    dist = _init(rank, world, port)
    from legion_b200.config import ModelConfig
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    from legion_b200.models.weights import Shard, random_weights
    from legion_b200.parallel.context import ParallelCtx
    from legion_b200.parallel.symm import SymmComm
    dev = torch.device("cuda", rank)
    cfg = ModelConfig(arch="qwen3moe", n_layer=3, hidden=512, vocab=2048, n_head=8, n_kv_head=2, head_dim=128,
                      n_expert=8, top_k=2, expert_ff=256)
    full = random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05)
    full = {k: (v.bfloat16() if v.dim() > 1 else v) for k, v in full.items()}
    w = {k: v.to(dev) for k, v in Shard(cfg, rank, world).shard_all(full).items()}
    symm = SymmComm(dist.group.WORLD, rank, world, dev, 1024, cfg.hidden) if comm_kind == "fused" else None
    pctx = ParallelCtx(rank, world, dist.group.WORLD, False, comm_kind, symm)
    eng = build_engine(cfg, weights=w, device=str(dev), pctx=pctx, start=False,
                       engine_cfg=EngineConfig(ctx_size=512, max_seqs=2, block_size=64, prefill_chunk=256, prefix_cache=False))
    prompt = torch.randint(0, 255, (200,), generator=torch.Generator().manual_seed(1)).tolist()
    s = eng.generate(GenerateRequest(prompt_tokens=prompt, sampling=SamplingParams(max_tokens=12, ignore_eos=True)))
    eng._drain(block=False)
    for _ in range(100):
        eng._admit()
        if not eng.running and len(eng.waiting) == 0:
            break
        eng.step()
    toks = s.collect().token_ids
    if symm is not None:
        symm.check()
    if rank == 0:
        torch.save({"tokens": toks, "graph_replays": eng._graphs.replays if eng._graphs else 0}, out_path)
    dist.barrier()
    dist.destroy_process_group()


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


@pytest.mark.parametrize("world", [2, 4])
def test_fused_all_reduce_norm(tmp_path, world):
    _need(world)
    out = str(tmp_path / "e.pt")
    mp.spawn(_comm_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    errs = torch.load(out)
    assert max(errs) < 0.08, errs


def test_tp_engine_fused_equals_nccl(tmp_path):
    _need(2)
    res = {}
    for kind in ("nccl", "fused"):
        out = str(tmp_path / f"{kind}.pt")
        mp.spawn(_engine_worker, args=(2, _free_port(), kind, out), nprocs=2, join=True)
        res[kind] = torch.load(out)
    assert len(res["fused"]["tokens"]) == 12
    assert res["fused"]["tokens"] == res["nccl"]["tokens"]
    assert res["fused"]["graph_replays"] > 0
