"""Data-parallel attention with expert parallelism as gloo processes on the CPU: each rank owns a share of the
sequences (attention, KV and recurrent state only for those) and a share of the routed experts; tokens meet their
experts inside each MoE layer. Output equals the single-process engine token for token."""
import socket

import pytest
import torch
import torch.multiprocessing as mp

from legion_b200.config import tiny_gqa_moe, tiny_hybrid_moe, tiny_mla_moe

CFGS = {"gqa_moe": tiny_gqa_moe, "hybrid": tiny_hybrid_moe, "mla": tiny_mla_moe}
ECFG = dict(ctx_size=512, max_seqs=4, block_size=16, prefill_chunk=96, prefix_cache=False)
BATCHES = (((150, 1),), ((40, 2), (33, 3), (61, 4)))   # one sequence (the other rank idles on a padding row), then three


# the same 150-token prompt three times (alone, beside another one, alone again): prefix hits must stay on its owner
REPEATS = (((150, 1),), ((40, 2), (150, 1)), ((150, 1), (33, 3)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _prompt(n, seed):
    return torch.randint(0, 255, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _run(eng, batches=BATCHES):
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    toks, owners = [], []
    for batch in batches:
        streams = [eng.generate(GenerateRequest(prompt_tokens=_prompt(n, s),
                                                sampling=SamplingParams(max_tokens=8, ignore_eos=True)))
                   for n, s in batch]
        eng._drain(block=False)
        for _ in range(300):
            eng._admit()
            owners += [s.owner if s.owner >= 0 else s.slot for s in eng.running]
            if not eng.running and len(eng.waiting) == 0:
                break
            eng.step()
        toks += [s.collect().token_ids for s in streams]
    return toks, sorted(set(owners))


def _worker(rank, world, port, name, out_path, prefix_cache=False):
    import datetime

    import torch.distributed as dist
    from legion_b200.engine.lm import EngineConfig, LmEngine
    from legion_b200.loaders.tokenizer import ByteTokenizer
    from legion_b200.models.decoder import Decoder
    from legion_b200.models.weights import Shard, random_weights
    from legion_b200.parallel.context import DpEpCtx
    torch.set_num_threads(2)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=120))
    cfg = CFGS[name]()
    full = random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05)
    w = Shard(cfg, rank, world, dp_attention=True).shard_all(full)
    assert w["l1.moe.gate_up"].shape[0] == cfg.n_expert // world       # experts split ...
    assert all(v.shape == full[k].shape for k, v in w.items() if ".moe.gate_up" not in k and ".moe.down" not in k)
    ec = EngineConfig(**dict(ECFG, prefix_cache=prefix_cache))
    model = Decoder(cfg, w, DpEpCtx(rank, world, dist.group.WORLD), max_position=ec.ctx_size + 8)
    eng = LmEngine(model, ByteTokenizer(cfg.vocab), ec, start=False)
    toks, slots = _run(eng, REPEATS if prefix_cache else BATCHES)
    if rank == 0:
        torch.save({"tokens": toks, "slots": slots, "hit_tokens": eng.radix.hit_tokens if eng.radix else 0},
                   out_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("name", ["gqa_moe", "hybrid", "mla"])
def test_dp_attention_equals_single(tmp_path, name):
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.models.weights import random_weights
    cfg = CFGS[name]()
    eng = build_engine(cfg, weights=random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05),
                       engine_cfg=EngineConfig(**ECFG), start=False)
    want, _ = _run(eng)
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(2, _free_port(), name, out), nprocs=2, join=True)
    got = torch.load(out)
    assert got["tokens"] == want
    assert len(got["slots"]) >= 2          # sequences landed on both owners


def test_dp_attention_prefix_cache_follows_the_owner(tmp_path):
    """With the prefix cache on, a prompt that hits cached blocks runs on the rank that computed them (the contents
    exist only there): same tokens as one process, and the hits are real."""
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.models.weights import random_weights
    cfg = CFGS["gqa_moe"]()
    eng = build_engine(cfg, weights=random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05),
                       engine_cfg=EngineConfig(**dict(ECFG, prefix_cache=True)), start=False)
    want, _ = _run(eng, REPEATS)
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(2, _free_port(), "gqa_moe", out, True), nprocs=2, join=True)
    got = torch.load(out)
    assert got["tokens"] == want
    assert got["hit_tokens"] >= 2 * 128            # the repeated prompt reused its 144 cached tokens twice
