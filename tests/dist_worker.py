"""Worker of the multi-GPU tests: one process per GPU, started by ``torch.distributed.run`` from
``test_comm_gpu.py``. Usage: ``dist_worker.py <case> <out_path>``. Every stage is logged to
``<out_path>.r<rank>.log`` and a watchdog dumps all stacks and exits if the case takes too long, so a stall shows
where it happened instead of running into the caller's limit."""
import datetime
import faulthandler
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

RANK = int(os.environ["RANK"])
WORLD = int(os.environ["WORLD_SIZE"])
CASE, OUT = sys.argv[1], sys.argv[2]
LOG = open(f"{OUT}.r{RANK}.log", "w", buffering=1)
T0 = time.time()
faulthandler.enable(LOG)
faulthandler.dump_traceback_later(int(os.environ.get("LB_TEST_WATCHDOG_S", "150")), exit=True, file=LOG)


def say(*a):
    print(f"[{time.time() - T0:7.2f}]", *a, file=LOG, flush=True)


def case_comm(dev):
    from legion_b200.ops import reference as ref
    from legion_b200.ops import sm100
    from legion_b200.parallel.symm import SymmComm
    H = 512
    comm = SymmComm(dist.group.WORLD, RANK, WORLD, dev, max_rows=2048, hidden=H, budget_ns=2_000_000_000)
    say("communicator up")
    torch.manual_seed(7)
    errs = []
    for T in (1, 16, 600, 2048):           # one-shot sizes and (world > 2) two-shot sizes
        parts = [(torch.randn(T, H, device=dev) * 0.5).bfloat16() for _ in range(WORLD)]     # same on every rank
        res = torch.randn(T, H, device=dev).bfloat16()
        w = torch.rand(H, device=dev) + 0.5
        slot = comm.next_partial(T, H)
        slot.copy_(parts[RANK])
        normed, summed = comm.all_reduce_add_norm(slot, res, w, 1e-6, 0.0)
        total = sum(p.float() for p in parts) + res.float()
        want_n, _ = ref.rmsnorm(total.bfloat16(), w, 1e-6)
        errs.append(float((summed.float() - total).abs().max()))
        errs.append(float((normed.float() - want_n.float()).abs().max()))
        comm.check()
        gathered = [torch.empty_like(summed) for _ in range(WORLD)]   # rank-order sums: same bits everywhere
        dist.all_gather(gathered, summed)
        assert all(torch.equal(g, gathered[0]) for g in gathered)
        say("rows", T, "ok")
    # decode-sized reduction that also emits the normalised rows NVFP4-encoded: same codes, scale bytes and row
    # scales as the stand-alone quantiser gives for the normalised rows
    for T in (3, 16, 64):
        parts = [(torch.randn(T, H, device=dev) * 0.5).bfloat16() for _ in range(WORLD)]
        res = torch.randn(T, H, device=dev).bfloat16()
        w = torch.rand(H, device=dev) + 0.5
        slot = comm.next_partial(T, H)
        slot.copy_(parts[RANK])
        normed, summed, xq = comm.all_reduce_add_norm(slot, res, w, 1e-6, 0.0, quant=True)
        total = sum(p.float() for p in parts) + res.float()
        errs.append(float((summed.float() - total).abs().max()))
        rq = sm100.nv4_quant_act(normed)
        assert torch.equal(xq.codes[:T], rq.codes) and torch.equal(xq.gscale[:T], rq.gscale[:T])
        assert torch.equal(xq.dequantize(), rq.dequantize())
        comm.check()
        say("quantising reduction rows", T, "ok")
    # the reduction sums this rank's weighted expert rows per token itself (no combine launch before it): every
    # rank owns a range of experts, rank 0 also brings a shared-expert row per token
    for T, k in ((16, 4), (1, 8), (50, 6)):
        E = 4 * WORLD
        ids = torch.randint(0, E, (T, k), device=dev, dtype=torch.int32)
        ys = [(torch.randn(T * k, H, device=dev) * 0.3).bfloat16() for _ in range(WORLD)]
        shared = (torch.randn(T, H, device=dev) * 0.3).bfloat16()
        res = torch.randn(T, H, device=dev).bfloat16()
        w = torch.rand(H, device=dev) + 0.5
        total = res.float()
        for r in range(WORLD):
            on = ((ids >= 4 * r) & (ids < 4 * r + 4)).reshape(T, k, 1).float()
            part = (ys[r].float().view(T, k, H) * on).sum(1) + (shared.float() if r == 0 else 0.0)
            total = total + part.bfloat16().float()
        pend = sm100.PendingCombine(ys[RANK], ids, 4 * RANK, 4 * RANK + 4, shared if RANK == 0 else None, T, H)
        normed, summed, xq = comm.all_reduce_add_norm(comm.next_partial(T, H), res, w, 1e-6, 0.0, quant=True, combine=pend)
        errs.append(float((summed.float() - total).abs().max()))
        want_n, _ = ref.rmsnorm(summed, w, 1e-6)
        errs.append(float((normed.float() - want_n.float()).abs().max()))
        rq = sm100.nv4_quant_act(normed)
        assert torch.equal(xq.codes[:T], rq.codes)
        comm.check()
        say("combine inside the reduction, rows", T, "ok")
    # GEMM epilogue writes straight into the slot, then the fused reduction
    x = (torch.randn(24, 256, device=dev) * 0.3).bfloat16()
    wts = [(torch.randn(H, 256, device=dev) * 0.05).bfloat16() for _ in range(WORLD)]
    res = torch.randn(24, H, device=dev).bfloat16()
    slot = comm.next_partial(24, H)
    sm100.linear(x, wts[RANK], out=slot)
    assert comm.owns(slot)
    _, summed = comm.all_reduce_add_norm(slot, res, None, 0.0, 0.0)
    want = sum(ref.linear(x, wt).float() for wt in wts) + res.float()
    errs.append(float((summed.float() - want).abs().max()))
    comm.end_step()
    comm.check()
    # all-gather -> GEMM in one kernel: every rank contributes its block of rows. Calls of different sizes run back
    # to back with no host synchronisation in between (a fast rank may start writing the next call's block while
    # a slower peer still copies this call's rows: the two alternating regions keep them apart); the gathered
    # rows are compared bit for bit afterwards.
    kept = []
    for it, T in enumerate((16, 300, 64, 1000, 16, 300, 7)):
        xs = (torch.randn(T, H, device=dev) * 0.3).bfloat16()          # same on every rank
        wq = (torch.randn(384, H, device=dev) * 0.05).bfloat16()
        row0, n, _ = comm.shard_rows(T)
        comm.shard_view(T).copy_(xs[row0:row0 + n])
        out, gathered = comm.all_gather_linear(T, wq)
        kept.append((T, xs, wq, out, gathered.clone()))
        if it == 3:      # a two-shot all-reduce in between shares the buffer but not the regions
            slot = comm.next_partial(600, H)
            slot.copy_((torch.randn(600, H, device=dev) * 0.5).bfloat16())
            comm.all_reduce_add_norm(slot, None, None, 0.0, 0.0)
    comm.check()
    for T, xs, wq, out, gathered in kept:
        assert torch.equal(gathered, xs), f"gathered rows differ at T={T}"
        errs.append(float((out.float() - ref.linear(xs, wq).float()).abs().max()))
        say("all-gather GEMM rows", T, "ok")
    assert sm100.Workspace.get(dev).check() == 0
    return {"errs": errs}


def case_comm_multimem(dev):
    """Two-shot reduction with the multimem form against the fp32 sum, and against the plain two-shot form's bits
    where both round alike is not required: the switch sums in fp32 and rounds once to bf16 before the residual."""
    from legion_b200.ops import reference as ref
    from legion_b200.parallel.symm import SymmComm
    H = 512
    comm = SymmComm(dist.group.WORLD, RANK, WORLD, dev, max_rows=2048, hidden=H, budget_ns=2_000_000_000)
    if not comm.mc_ptr:
        return {"skipped": "the symmetric buffer has no NVLink multicast mapping on this box"}
    say("multicast mapping", hex(comm.mc_ptr))
    torch.manual_seed(11)
    errs = []
    for T in (600, 2048, 513):
        parts = [(torch.randn(T, H, device=dev) * 0.5).bfloat16() for _ in range(WORLD)]
        res = torch.randn(T, H, device=dev).bfloat16()
        w = torch.rand(H, device=dev) + 0.5
        slot = comm.next_partial(T, H)
        slot.copy_(parts[RANK])
        normed, summed = comm.all_reduce_add_norm(slot, res, w, 1e-6, 0.0)
        total = sum(p.float() for p in parts) + res.float()
        errs.append(float((summed.float() - total).abs().max()))
        want_n, _ = ref.rmsnorm(summed, w, 1e-6)
        errs.append(float((normed.float() - want_n.float()).abs().max()))
        comm.check()
        gathered = [torch.empty_like(summed) for _ in range(WORLD)]
        dist.all_gather(gathered, summed)
        assert all(torch.equal(g, gathered[0]) for g in gathered)      # every rank holds the same rows
        say("multimem rows", T, "ok", errs[-2])
    comm.end_step()
    comm.check()
    return {"errs": errs}


def case_ep(dev):
    from legion_b200.ops import reference as ref
    from legion_b200.ops import sm100
    from legion_b200.parallel.ep import EpDispatcher
    E, k, F, H = 8, 2, 256, 512
    ep = EpDispatcher(dist.group.WORLD, RANK, WORLD, dev, E, k, H, F, max_tokens=64, budget_ns=2_000_000_000)
    say("dispatcher up, tile", ep.bn, "capacity", ep.cap)
    g = torch.Generator().manual_seed(3)
    gu_all = (torch.randn(E, 2 * F, H, generator=g) * 0.05).bfloat16()
    dn_all = (torch.randn(E, H, F, generator=g) * 0.05).bfloat16()
    per = E // WORLD
    gu = gu_all[RANK * per:(RANK + 1) * per].to(dev).contiguous()
    dn = dn_all[RANK * per:(RANK + 1) * per].to(dev).contiguous()
    errs = []
    for it, T in enumerate((5, 64, 33, 1)):       # every rank brings different tokens
        gg = torch.Generator().manual_seed(100 + it * 8 + RANK)
        x = (torch.randn(T, H, generator=gg) * 0.5).bfloat16().to(dev)
        logits = torch.randn(T, E, generator=gg).to(dev)
        ids, wts = sm100.router_topk(logits, k)
        y = ep.forward(x, ids, wts, gu, dn)
        ep.check()
        want = ref.moe_experts(x.cpu(), ids.cpu(), wts.cpu(), gu_all, dn_all, F)
        errs.append(float((y.cpu().float() - want.float()).abs().max()))
        say("tokens", T, "err", errs[-1])
    assert sm100.Workspace.get(dev).check() == 0
    all_errs = [None] * WORLD
    dist.all_gather_object(all_errs, errs)
    return {"errs": [e for es in all_errs for e in es]}


def case_engine(dev, comm_kind):
    from legion_b200.config import ModelConfig
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    from legion_b200.models.weights import Shard, random_weights
    from legion_b200.parallel.context import ParallelCtx
    from legion_b200.parallel.symm import SymmComm
    cfg = ModelConfig(arch="qwen3moe", n_layer=3, hidden=512, vocab=2048, n_head=8, n_kv_head=2, head_dim=128,
                      n_expert=8, top_k=2, expert_ff=256)
    full = random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05)
    full = {k: (v.bfloat16() if v.dim() > 1 else v) for k, v in full.items()}
    w = {k: v.to(dev) for k, v in Shard(cfg, RANK, WORLD).shard_all(full).items()}
    symm = None
    tail = comm_kind == "tail"          # o-proj GEMM and its all-reduce as one kernel
    if tail:
        comm_kind = "fused"
    if comm_kind == "fused":
        symm = SymmComm(dist.group.WORLD, RANK, WORLD, dev, 1024, cfg.hidden, budget_ns=2_000_000_000)
    pctx = ParallelCtx(RANK, WORLD, dist.group.WORLD, False, comm_kind, symm, gemm_tail=tail)
    eng = build_engine(cfg, weights=w, device=str(dev), pctx=pctx, start=False,
                       engine_cfg=EngineConfig(ctx_size=512, max_seqs=2, block_size=64, prefill_chunk=256,
                                               prefix_cache=False))
    say("engine built")
    prompt = torch.randint(0, 255, (200,), generator=torch.Generator().manual_seed(1)).tolist()
    s = eng.generate(GenerateRequest(prompt_tokens=prompt, sampling=SamplingParams(max_tokens=12, ignore_eos=True)))
    eng._drain(block=False)
    for i in range(100):
        eng._admit()
        if not eng.running and len(eng.waiting) == 0:
            break
        eng.step()
        if symm is not None:
            symm.check()
        say("step", i)
    toks = s.collect().token_ids
    replays = eng._graphs.replays if eng._graphs else 0
    eng.shutdown()          # graphs that captured NCCL collectives go before the process group does
    return {"tokens": toks, "graph_replays": replays}


def case_engine_nv4(dev, comm_kind):
    """The serving layout of the NVFP4 hybrid configuration on several GPUs: attention and Gated DeltaNet heads split
    by rank, routed experts whole per rank (NVFP4, native W4A4 GEMMs), the shared expert whole on rank (layer mod
    world) stacked behind that rank's experts, decode steps from CUDA graphs. ``fused``: quantising pushed-line
    reduction with the MoE combine inside; ``nccl``: NCCL all-reduce + separate kernels. Returns the first decode
    step's logits too, so that runs whose reduction order differs (more than two ranks) can be compared by value."""
    from legion_b200.config import ModelConfig
    from legion_b200.engine.lm import EngineConfig, LmEngine
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    from legion_b200.loaders.tokenizer import ByteTokenizer
    from legion_b200.models.decoder import Decoder, place_shared_expert, quantize_moe_layer_nvfp4
    from legion_b200.models.weights import Shard, random_weights
    from legion_b200.parallel.context import ParallelCtx
    from legion_b200.parallel.symm import SymmComm
    kinds = ["gdn", "gdn", "attn", "gdn"]
    cfg = ModelConfig(arch="qwen35moe", n_layer=4, hidden=512, vocab=2048, n_head=8, n_kv_head=2, head_dim=128,
                      layer_kinds=kinds, gated_attn=True, rope_dim=64, gdn_k_heads=8, gdn_v_heads=16, gdn_k_dim=128,
                      gdn_v_dim=128, gdn_conv=4, n_expert=16, top_k=4, expert_ff=256, shared_ff=256, shared_gate=True)
    full = random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05)
    full = {k: (v.bfloat16() if v.dim() > 1 and not k.endswith("conv_w") else v) for k, v in full.items()}
    sh = Shard(cfg, RANK, WORLD, expert_parallel=True, shared_whole=True)
    w = {k: v.to(dev) for k, v in sh.shard_all(full).items()}
    for il in range(cfg.n_layer):
        place_shared_expert(w, f"l{il}", il, cfg, RANK, WORLD)
        quantize_moe_layer_nvfp4(w, f"l{il}")
    symm = SymmComm(dist.group.WORLD, RANK, WORLD, dev, 1024, cfg.hidden, budget_ns=2_000_000_000) \
        if comm_kind == "fused" else None
    pctx = ParallelCtx(RANK, WORLD, dist.group.WORLD, True, comm_kind, symm)
    model = Decoder(cfg, w, pctx, max_position=520)
    model.fuse_gdn_in_proj()
    if comm_kind == "fused":
        assert model.split_head()           # vocabulary-split LM head: greedy picks by (value, id) pair exchange
    eng = LmEngine(model, ByteTokenizer(cfg.vocab), EngineConfig(ctx_size=512, max_seqs=4, block_size=64, prefill_chunk=256,
                                                                 prefix_cache=False, device=str(dev)), start=False)
    say("engine built")
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 255, (n,), generator=g).tolist() for n in (200, 70, 131)]
    streams = [eng.generate(GenerateRequest(prompt_tokens=p, sampling=SamplingParams(max_tokens=10, ignore_eos=True)))
               for p in prompts]
    eng._drain(block=False)
    for i in range(200):
        eng._admit()
        if not eng.running and len(eng.waiting) == 0:
            break
        eng.step()
        if symm is not None:
            symm.check()
    toks = [s.collect().token_ids for s in streams]
    replays = eng._graphs.replays if eng._graphs else 0
    # one more eager decode-sized forward over fixed rows: logits by value
    seq = eng.prepare(GenerateRequest(prompt_tokens=prompts[1], sampling=SamplingParams(max_tokens=2, ignore_eos=True)))
    eng.waiting.push(seq)
    eng._admit()
    b = eng.build_batch([(seq, 0, len(prompts[1]))])
    logits = eng.model.forward(b, eng.kv, eng.states).logits.float().cpu()
    from legion_b200.ops import sm100
    assert sm100.Workspace.get(dev).check() == 0
    eng.shutdown()
    return {"tokens": toks, "graph_replays": replays, "logits": logits}


def case_peer_experts(dev):
    """Experts sharded over the ranks' symmetric memory; a rank's grouped GEMM streams a PEER's expert tiles over
    NVLink with plain (non-multicast) TMA loads. Every rank computes the whole MoE layer from all shards."""
    from legion_b200.ops import reference as ref
    from legion_b200.ops import sm100
    from legion_b200.residency.experts import PeerExperts
    E, k, F, H = 8, 2, 256, 512
    g = torch.Generator().manual_seed(5)
    gu_all = (torch.randn(E, 2 * F, H, generator=g) * 0.05).bfloat16()
    dn_all = (torch.randn(E, H, F, generator=g) * 0.05).bfloat16()
    per = E // WORLD
    pe = PeerExperts(gu_all[RANK * per:(RANK + 1) * per].to(dev).contiguous(),
                     dn_all[RANK * per:(RANK + 1) * per].to(dev).contiguous(), dist.group.WORLD, RANK, WORLD)
    say("peer shards mapped")
    errs = []
    for T in (7, 100):
        gg = torch.Generator().manual_seed(40 + T)
        x = (torch.randn(T, H, generator=gg) * 0.5).bfloat16().to(dev)
        ids, wts = sm100.router_topk(torch.randn(T, E, generator=gg).to(dev), k)
        y = torch.zeros(T, H, device=dev)
        for r in range(WORLD):
            gu, dn = pe.views(r)
            y += sm100.moe_experts(x, ids, wts, gu, dn, F, e_lo=pe.expert_range(r)[0]).float()
        torch.cuda.synchronize()
        want = ref.moe_experts(x.cpu(), ids.cpu(), wts.cpu(), gu_all, dn_all, F)
        errs.append(float((y.cpu() - want.float()).abs().max()))
        say("tokens", T, "err", errs[-1])
    assert sm100.Workspace.get(dev).check() == 0
    dist.barrier()          # no rank frees its shard while a peer may still read it
    return {"errs": errs}


def case_engine_dp(dev):
    """Data-parallel attention + expert-parallel exchange on GPUs against one GPU holding the whole model."""
    from legion_b200.config import ModelConfig
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    from legion_b200.models.weights import Shard, random_weights
    from legion_b200.parallel.context import DpEpCtx
    from legion_b200.parallel.ep import EpDispatcher
    cfg = ModelConfig(arch="qwen3moe", n_layer=3, hidden=512, vocab=2048, n_head=8, n_kv_head=2, head_dim=128,
                      n_expert=8, top_k=2, expert_ff=256)
    full = random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05)
    full = {k: (v.bfloat16() if v.dim() > 1 else v) for k, v in full.items()}
    ecfg = dict(ctx_size=512, max_seqs=4, block_size=64, prefill_chunk=128, max_batch_tokens=256, prefix_cache=False)

    def run(eng):
        prompts = [torch.randint(0, 255, (n,), generator=torch.Generator().manual_seed(sd)).tolist()
                   for n, sd in ((200, 1), (70, 2), (131, 3))]
        streams = [eng.generate(GenerateRequest(prompt_tokens=p, sampling=SamplingParams(max_tokens=10, ignore_eos=True)))
                   for p in prompts]
        eng._drain(block=False)
        for i in range(200):
            eng._admit()
            if not eng.running and len(eng.waiting) == 0:
                break
            eng.step()
        return [s.collect().token_ids for s in streams]

    single = build_engine(cfg, weights={k: v.to(dev) for k, v in full.items()}, device=str(dev), start=False,
                          engine_cfg=EngineConfig(cuda_graphs=False, **ecfg))
    want = run(single)
    single.shutdown()
    say("single-GPU run done")
    w = {k: v.to(dev) for k, v in Shard(cfg, RANK, WORLD, dp_attention=True).shard_all(full).items()}
    ep = EpDispatcher(dist.group.WORLD, RANK, WORLD, dev, cfg.n_expert, cfg.top_k, cfg.hidden, cfg.expert_ff,
                      max_tokens=256, budget_ns=2_000_000_000)
    eng = build_engine(cfg, weights=w, device=str(dev), pctx=DpEpCtx(RANK, WORLD, dist.group.WORLD, ep), start=False,
                       engine_cfg=EngineConfig(**ecfg))
    say("dp engine built")
    got = run(eng)
    ep.check()
    replays = eng._graphs.replays if eng._graphs else 0
    eng.shutdown()
    return {"tokens": got, "single": want, "graph_replays": replays}


def case_pp(dev):
    """Pipeline stages over NCCL send / recv: same tokens as the whole model on one GPU."""
    from legion_b200.config import ModelConfig
    from legion_b200.engine.lm import EngineConfig, LmEngine, build_engine
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    from legion_b200.loaders.tokenizer import ByteTokenizer
    from legion_b200.models.decoder import Decoder
    from legion_b200.models.weights import layer_of, random_weights
    from legion_b200.parallel.pipeline import PipeStage
    cfg = ModelConfig(arch="qwen3moe", n_layer=4, hidden=512, vocab=2048, n_head=8, n_kv_head=2, head_dim=128,
                      n_expert=8, top_k=2, expert_ff=256)
    full = random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05)
    full = {k: (v.bfloat16() if v.dim() > 1 else v) for k, v in full.items()}
    ecfg = dict(ctx_size=1024, max_seqs=2, block_size=64, prefill_chunk=512, prefix_cache=False)
    prompt = torch.randint(0, 255, (300,), generator=torch.Generator().manual_seed(1)).tolist()

    def run(eng):
        s = eng.generate(GenerateRequest(prompt_tokens=prompt, sampling=SamplingParams(max_tokens=10, ignore_eos=True)))
        eng._drain(block=False)
        for _ in range(100):
            eng._admit()
            if not eng.running and len(eng.waiting) == 0:
                break
            eng.step()
        return s.collect().token_ids

    res = {}
    for micro in (4096, 128):
        pipe = PipeStage(RANK, WORLD, dist.group.WORLD, cfg.n_layer, micro_tokens=micro)
        w = {k: v.to(dev) for k, v in full.items() if layer_of(k) is None or pipe.owns(layer_of(k))}
        model = Decoder(cfg, w, None, max_position=1032, pipe=pipe)
        eng = LmEngine(model, ByteTokenizer(cfg.vocab), EngineConfig(device=str(dev), **ecfg), start=False)
        res[f"pp_micro{micro}"] = run(eng)
        res[f"chunks_micro{micro}"] = pipe.stats["micro_chunks"]
        say("pipeline run, micro", micro, "chunks", pipe.stats["micro_chunks"])
    if RANK == 0:
        eng = build_engine(cfg, weights={k: v.to(dev) for k, v in full.items()}, device=str(dev), start=False,
                           engine_cfg=EngineConfig(cuda_graphs=False, **ecfg))
        res["single"] = run(eng)
    return res


def main():
    torch.cuda.set_device(RANK)
    dev = torch.device("cuda", RANK)
    dist.init_process_group("nccl", timeout=datetime.timedelta(seconds=60), device_id=dev)
    say("process group up")
    if CASE == "comm":
        res = case_comm(dev)
    elif CASE == "comm_multimem":
        res = case_comm_multimem(dev)
    elif CASE == "ep":
        res = case_ep(dev)
    elif CASE == "pp":
        res = case_pp(dev)
    elif CASE == "peer_experts":
        res = case_peer_experts(dev)
    elif CASE == "engine_dp":
        res = case_engine_dp(dev)
    elif CASE in ("engine_nv4_nccl", "engine_nv4_fused"):
        res = case_engine_nv4(dev, CASE.split("_")[2])
    elif CASE in ("engine_nccl", "engine_fused", "engine_tail"):
        res = case_engine(dev, CASE.split("_")[1])
    else:
        raise SystemExit(f"unknown case {CASE}")
    torch.cuda.synchronize()
    if RANK == 0:
        torch.save(res, OUT)
    say("result saved")
    dist.barrier()
    say("barrier passed")
    faulthandler.cancel_dump_traceback_later()
    faulthandler.dump_traceback_later(20, exit=True, file=LOG)
    dist.destroy_process_group()
    faulthandler.cancel_dump_traceback_later()
    say("done")


if __name__ == "__main__":
    main()
