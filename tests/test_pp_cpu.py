"""Pipeline-parallel stages as gloo processes on the CPU: layers split over 2 / 3 ranks, residual by send / recv,
long prompt chunks cut into micro-chunks. Output equals the single-process engine token for token."""
import socket

import pytest
import torch
import torch.multiprocessing as mp

from legion_b200.config import tiny_gqa_moe, tiny_hybrid_moe

CFGS = {"gqa_moe": tiny_gqa_moe, "hybrid": tiny_hybrid_moe}
ECFG = dict(ctx_size=512, max_seqs=4, block_size=16, prefill_chunk=160, prefix_cache=False)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _prompt(n, seed):
    return torch.randint(0, 255, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _worker(rank, world, port, name, out_path):
    import datetime

    import torch.distributed as dist
    from legion_b200.engine.lm import EngineConfig, LmEngine
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    from legion_b200.loaders.tokenizer import ByteTokenizer
    from legion_b200.models.decoder import Decoder
    from legion_b200.models.weights import random_weights
    from legion_b200.parallel.pipeline import PipeStage
    torch.set_num_threads(2)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=120))
    cfg = CFGS[name]()
    pipe = PipeStage(rank, world, dist.group.WORLD, cfg.n_layer, micro_tokens=48, decode_groups=2)
    full = random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05)
    # a stage keeps its own layers, the embedding (first stage; tied heads) and the head (last stage)
    w = {k: v for k, v in full.items()
         if not k.startswith("l") or not k[1].isdigit() or pipe.owns(int(k[1:k.index(".")]))}
    ec = EngineConfig(**ECFG)
    model = Decoder(cfg, w, None, max_position=ec.ctx_size + 8, pipe=pipe)
    eng = LmEngine(model, ByteTokenizer(cfg.vocab), ec, start=False)
    assert set(eng.kv.k) == {il for il in cfg.kv_layers() if pipe.owns(il)}
    toks = []
    # one long prompt alone (micro-chunked), two together, then four together (their decode steps travel the stages
    # as two groups of two)
    for batch in (((150, 1),), ((40, 2), (33, 3)), ((20, 4), (25, 5), (18, 6), (30, 7))):
        streams = [eng.generate(GenerateRequest(prompt_tokens=_prompt(n, s),
                                                sampling=SamplingParams(max_tokens=8, ignore_eos=True)))
                   for n, s in batch]
        eng._drain(block=False)
        for _ in range(200):
            eng._admit()
            if not eng.running and len(eng.waiting) == 0:
                break
            eng.step()
        toks += [s.collect().token_ids for s in streams]
    if rank == 0:
        torch.save({"tokens": toks, "micro": pipe.stats["micro_chunks"], "sends": pipe.stats["sends"],
                    "groups": pipe.stats["decode_groups"],
                    "bounds": pipe.bounds}, out_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("name,world", [("gqa_moe", 2), ("hybrid", 2), ("gqa_moe", 3)])
def test_pipeline_equals_single(tmp_path, name, world):
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.models.weights import random_weights
    cfg = CFGS[name]()
    eng = build_engine(cfg, weights=random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05),
                       engine_cfg=EngineConfig(**ECFG))
    want = [eng.generate_text(tokens=_prompt(n, s), max_tokens=8, ignore_eos=True).token_ids
            for n, s in ((150, 1), (40, 2), (33, 3), (20, 4), (25, 5), (18, 6), (30, 7))]
    eng.shutdown()
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(world, _free_port(), name, out), nprocs=world, join=True)
    got = torch.load(out)
    assert got["tokens"] == want
    assert got["micro"] >= 3           # the 150-token prompt went through as micro-chunks of 48
    assert got["groups"] >= 4          # decode steps of four sequences went through as two groups
    assert got["sends"] > 0 and got["bounds"][-1] == cfg.n_layer


def test_layer_split_rules():
    from legion_b200.parallel.pipeline import split_layers
    assert split_layers(48, 8) == [0, 6, 12, 18, 24, 30, 36, 42, 48]
    assert split_layers(61, 8)[-1] == 61 and len(split_layers(61, 8)) == 9
    assert split_layers(10, 3, last_extra=2) == [0, 5, 9, 10]
    assert split_layers(10, 2, layer_split=[7, 3]) == [0, 7, 10]
    with pytest.raises(ValueError):
        split_layers(10, 2, layer_split=[7, 2])
