"""Tensor / expert parallel ranks as gloo processes on the CPU: TP=n output equals TP=1 token for token
(the reference tests its TP the same way: ranks as threads over loopback, tests/qwen4_tp_net.rs)."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

from legion_b200.config import tiny_dense, tiny_gqa_moe, tiny_hybrid_moe

CFGS = {"gqa_moe": tiny_gqa_moe, "hybrid": tiny_hybrid_moe, "dense": tiny_dense}


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _prompt(n, seed):
    return torch.randint(0, 255, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _worker(rank, world, port, name, ep, out_path):
    import datetime

    import torch.distributed as dist
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.models.weights import Shard, random_weights
    from legion_b200.parallel.context import ParallelCtx
    torch.set_num_threads(2)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=120))
    cfg = CFGS[name]()
    full = random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05)
    w = Shard(cfg, rank, world, expert_parallel=ep).shard_all(full)
    pctx = ParallelCtx(rank, world, dist.group.WORLD, expert_parallel=ep, comm="nccl")
    eng = build_engine(cfg, weights=w, pctx=pctx,
                       engine_cfg=EngineConfig(ctx_size=256, max_seqs=2, block_size=16, prefill_chunk=64, prefix_cache=False),
                       start=False)
    # SPMD: every rank drives its own engine loop with the same requests and makes the same decisions
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    streams = [eng.generate(GenerateRequest(prompt_tokens=_prompt(90, s), sampling=SamplingParams(max_tokens=10, ignore_eos=True)))
               for s in (1, 2)]
    eng._drain(block=False)
    for _ in range(200):
        eng._admit()
        if not eng.running and len(eng.waiting) == 0:
            break
        eng.step()
    toks = [s.collect().token_ids for s in streams]
    if rank == 0:
        torch.save({"tokens": toks, "all_reduces": pctx.stats["all_reduce"]}, out_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("name,world,ep", [("gqa_moe", 2, False), ("gqa_moe", 2, True), ("hybrid", 2, False), ("dense", 2, False)])
def test_tp_equals_single(tmp_path, name, world, ep):
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.models.weights import random_weights
    cfg = CFGS[name]()
    eng = build_engine(cfg, weights=random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05),
                       engine_cfg=EngineConfig(ctx_size=256, max_seqs=2, block_size=16, prefill_chunk=64, prefix_cache=False))
    want = [eng.generate_text(tokens=_prompt(90, s), max_tokens=10, ignore_eos=True).token_ids for s in (1, 2)]
    eng.shutdown()
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(world, _free_port(), name, ep, out), nprocs=world, join=True)
    got = torch.load(out)
    assert got["tokens"] == want
    assert got["all_reduces"] > 0


def test_shard_shapes_cover_the_full_weights():
    from legion_b200.models.weights import Shard, random_weights, weight_shapes
    cfg = tiny_hybrid_moe()
    full = random_weights(cfg, "cpu", torch.float32, seed=0)
    for world in (2, 4):
        shards = [Shard(cfg, r, world).shard_all(full) for r in range(world)]
        for k, v in full.items():
            n_local = sum(s[k].numel() for s in shards)
            if k.endswith("attn.qkv") and cfg.n_kv_head < world:
                assert n_local > v.numel()                                # kv heads replicated
                continue
            assert n_local in (v.numel(), v.numel() * world), k       # split exactly once, or mirrored
        ep = [Shard(cfg, r, world, expert_parallel=True) for r in range(world)]
        assert [e.expert_range() for e in ep] == [(r * 8 // world, (r + 1) * 8 // world) for r in range(world)]


def _serve_worker(rank, world, port, out_path):
    import datetime
    import time

    import torch.distributed as dist
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    from legion_b200.models.weights import Shard, random_weights
    from legion_b200.parallel import spmd
    from legion_b200.parallel.context import ParallelCtx
    torch.set_num_threads(2)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=120))
    cfg = CFGS["gqa_moe"]()
    full = random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05)
    pctx = ParallelCtx(rank, world, dist.group.WORLD, False, "nccl")
    eng = build_engine(cfg, weights=Shard(cfg, rank, world).shard_all(full), pctx=pctx, start=False,
                       engine_cfg=EngineConfig(ctx_size=256, max_seqs=2, block_size=16, prefill_chunk=64, prefix_cache=False))
    spmd.attach(eng, rank, world, timeout_s=60)
    eng.start()
    if rank == 0:
        # requests arrive only at rank 0, at different times; one is cancelled mid-way
        a = eng.generate(GenerateRequest(prompt_tokens=_prompt(90, 1), sampling=SamplingParams(max_tokens=10, ignore_eos=True)))
        time.sleep(0.3)
        b = eng.generate(GenerateRequest(prompt_tokens=_prompt(90, 2), sampling=SamplingParams(max_tokens=10, ignore_eos=True)))
        c = eng.generate(GenerateRequest(prompt_tokens=_prompt(50, 3), sampling=SamplingParams(max_tokens=200, ignore_eos=True)))
        n = 0
        for ev in c:
            if ev.kind == "text":
                n += 1
                if n == 2:
                    c.cancel()
        torch.save({"tokens": [a.collect().token_ids, b.collect().token_ids], "cancelled_after": n}, out_path)
        eng.shutdown()          # broadcasts the shutdown message
    else:
        spmd.follower_wait(eng)
    dist.destroy_process_group()


def test_lock_step_serving_over_two_ranks(tmp_path):
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.models.weights import random_weights
    cfg = CFGS["gqa_moe"]()
    eng = build_engine(cfg, weights=random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05),
                       engine_cfg=EngineConfig(ctx_size=256, max_seqs=2, block_size=16, prefill_chunk=64, prefix_cache=False))
    want = [eng.generate_text(tokens=_prompt(90, s), max_tokens=10, ignore_eos=True).token_ids for s in (1, 2)]
    eng.shutdown()
    out = str(tmp_path / "serve.pt")
    mp.spawn(_serve_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    got = torch.load(out)
    assert got["tokens"] == want
    assert 2 <= got["cancelled_after"] < 200


def _leaver(rank, world, port, out_path):
    """Rank 1 leaves between steps (no collective of its own in flight); rank 0's next collective must end with an
    error within the group's timeout instead of hanging, and the error is what the host sees."""
    import datetime
    import time

    import torch.distributed as dist
    from legion_b200.parallel.context import ParallelCtx
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=8))
    pctx = ParallelCtx(rank, world, dist.group.WORLD, comm="nccl")
    x = torch.ones(4, 8)
    y = pctx.all_reduce(x.clone())                    # step 1: both ranks
    assert float(y[0, 0]) == world
    dist.barrier()
    if rank == 1:
        os._exit(0)                                   # gone before step 2
    t0 = time.time()
    err = None
    try:
        pctx.all_reduce(x.clone())                    # step 2: the peer never joins
    except Exception as e:                            # noqa: BLE001
        err = f"{type(e).__name__}: {e}"
    torch.save({"error": err, "seconds": time.time() - t0}, out_path)
    os._exit(0)


def test_a_rank_that_leaves_ends_the_next_collective_with_an_error(tmp_path):
    out = str(tmp_path / "r0.pt")
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_leaver, args=(r, 2, (port := _free_port()) if r == 0 else port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=90)
        assert not p.is_alive(), "a rank hung after its peer left"
    got = torch.load(out)
    assert got["error"] is not None and got["seconds"] < 30, got
