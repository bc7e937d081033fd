#!/usr/bin/env python
"""Headline benchmark: decode tokens/s at 1 / 16 / 64 concurrent users and tokens/s of a 32K-token prefill, on one of
the named model configurations, random-init weights and synthetic token ids, over N GPUs of one node.

    python bench.py --gpus N --steps K --warmup W [--config 3]      (N > 1: launched by torch.distributed.run)

Configurations (``--config``):
  3  (default) 80B-A3B-shape hybrid MoE, experts in NVFP4 (native W4A4 tensor-core path): 48 layers, 3:1 Gated
     DeltaNet to gated attention, 512 experts top-10 + shared expert, 1K-token prompts for the decode rows.
  2  30B-A3B-shape MoE in bf16: 48 layers, 128 experts top-8, 8K-token prompts.
  5  dense 27B-shape model in bf16, 1K-token prompts.
The ONE parsed number (``value``) is decode tokens/s at 16 users of the selected configuration; the other rows of
the grid (1 and 64 users, 32K prefill) are under ``extra``.

What is timed
  value        K decode steps of the whole batch, device-timed with CUDA events around K replays of the captured
               decode-step graph (every kernel of the step: all layers, LM head, arg-max), max over ranks; the
               K-step region is repeated ``--repeats`` times and the median is reported (min / max under extra).
               A step streams several GB of weights and state, far more than L2, so no L2 flush is needed.
  e2e          the same K steps through the public engine API (LmEngine.generate streams): each step packs that
               step's token ids / positions / block tables in pinned host memory, copies them to the device,
               replays the graph and reads the picked tokens back. Wall clock on rank 0.
  prefill      one prompt of ``--prefill-len`` tokens through the engine in chunks, device-timed to its first token.
``--impl reference`` reports that the reference cannot be built here (no Rust toolchain, empty ggml submodule).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time


def reference_arm():
    print(json.dumps({"impl": "reference",
                      "unavailable": "reference is a Rust crate over a ggml submodule that is empty here; no cargo/rustc "
                                     "in the image, so it cannot be installed or run (pip install of the reference tree has "
                                     "no Python package to build)"}))
    return 0


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.rows = []
        self._stop = threading.Event()
        self._t = None

    def start(self):
        def loop():
            while not self._stop.is_set():
                try:
                    out = subprocess.run(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.idx)], capture_output=True, text=True, timeout=5).stdout
                    for line in out.strip().splitlines():
                        self.rows.append([c.strip() for c in line.split(",")])
                except Exception:
                    pass
                self._stop.wait(0.1)
        self._t = threading.Thread(target=loop, daemon=True)
        self._t.start()

    def stop(self):
        self._stop.set()
        if self._t:
            self._t.join(timeout=6)
        sm, mx, reasons = [], 0.0, set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx = max(mx, float(r[2]))
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            except (ValueError, IndexError):
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


CONFIGS = {
    2: dict(model="qwen3-30b-a3b", prompt_len=8192, weights="bf16", dtype="bf16"),
    3: dict(model="qwen35-80b-a3b", prompt_len=1024, weights="nvfp4", dtype="nvfp4 experts (W4A4), bf16 elsewhere"),
    4: dict(model="deepseek-671b", prompt_len=1024, weights="fp8",
            dtype="fp8 (block-scaled e4m3 weights, e4m3 activations on the projections and experts), bf16 elsewhere"),
    5: dict(model="dense-27b", prompt_len=1024, weights="bf16", dtype="bf16"),
}


def build_model(a, cfg, dev, pctx, shard, weights_mode):
    """Random-init weights generated on the device; NVFP4 configurations are folded and quantised layer by layer
    while they are generated (their bf16 form would not fit one GPU)."""
    import torch
    from legion_b200.models.decoder import (Decoder, place_shared_expert, quantize_moe_layer_fp8,
                                            quantize_moe_layer_nvfp4)
    from legion_b200.models.weights import layer_of, random_weights
    world = pctx.world
    post = None
    if weights_mode == "nvfp4":
        def post(name, out):
            # the last expert tensor of a layer has arrived: stack the shared expert behind the routed ones
            # (single GPU) and encode the layer
            il = layer_of(name)
            if il is None or not cfg.is_moe_layer(il):
                return
            last = "moe.sh_gate" if (cfg.shared_ff > 0 and cfg.shared_gate) else ("moe.sh_down" if cfg.shared_ff > 0
                                                                                   else "moe.down")
            if not name.endswith(last):
                return
            p = f"l{il}"
            if not a.no_fold and (world == 1 or (shard is not None and shard.shared_whole)):
                place_shared_expert(out, p, il, cfg, pctx.rank, world)
            quantize_moe_layer_nvfp4(out, p, native=not a.nvfp4_expand)
    if weights_mode == "fp8":
        from legion_b200.ops.sm100 import Fp8Weight

        def post(name, out):
            # every projection is re-encoded to block-scaled e4m3 as soon as it has been generated (the bf16 form
            # of a 671B model does not fit the GPUs)
            t = out[name]
            leaf = name.split(".", 1)[1] if "." in name else name
            leaf = leaf.replace("l.", "", 1) if name.startswith("mtp") and leaf.startswith("l.") else leaf
            il = layer_of(name)
            if il is not None and cfg.is_moe_layer(il) and leaf.startswith("moe.") and not name.startswith("mtp"):
                # a routed layer: when its last expert tensor has arrived, the shared expert is stacked behind this
                # rank's routed experts (or dropped, on the ranks that do not keep it) and the layer is encoded
                last = "moe.sh_gate" if (cfg.shared_ff > 0 and cfg.shared_gate) else (
                    "moe.sh_down" if cfg.shared_ff > 0 else "moe.down")
                if leaf == last:
                    if not a.no_fold and (world == 1 or (shard is not None and shard.shared_whole)):
                        place_shared_expert(out, f"l{il}", il, cfg, pctx.rank, world)
                    quantize_moe_layer_fp8(out, f"l{il}")
                return
            if leaf not in Decoder.FP8_LEAVES or not isinstance(t, torch.Tensor) or t.dtype != torch.bfloat16:
                return
            if not a.fp8_all and not leaf.startswith(("mlp.", "moe.")):
                return      # the small attention projections stay bf16: no activation encoding in front of them
            rows, K = t.shape[-2], t.shape[-1]
            if K % 128 or rows % 128 or (leaf.endswith("gate_up") and (rows // 2) % 128):
                return
            out[name] = Fp8Weight.quantize(t)
    weights = random_weights(cfg, dev, torch.bfloat16, seed=0, shard=shard, post=post)
    torch.cuda.synchronize()
    return weights


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--config", type=int, default=3, choices=sorted(CONFIGS))
    ap.add_argument("--users", type=int, default=16, help="users of the headline row")
    ap.add_argument("--grid", default="1,64", help="other user counts reported under extra ('' = none)")
    ap.add_argument("--prompt-len", type=int, default=0, help="prompt length of the decode rows (0 = the config's)")
    ap.add_argument("--prefill-len", type=int, default=32768, help="length of the single-prompt prefill row (0 = skip)")
    ap.add_argument("--repeats", type=int, default=5, help="how often the K-step timed region is repeated")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--moe", default="auto", choices=["auto", "tp", "ep"],
                    help="N > 1: slice every expert's FFN rows over the ranks (tp) or keep whole experts per rank "
                         "with mirrored tokens, partial outputs meeting in the layer's reduction (ep). auto: ep "
                         "from 4 GPUs for bf16 experts, always for NVFP4 experts")
    ap.add_argument("--no-fold", action="store_true", help="keep the shared expert as a dense FFN of its own")
    ap.add_argument("--fp8-all", action="store_true",
                    help="config 4: also keep the attention projections in FP8 (default: FFNs and experts only)")
    ap.add_argument("--no-head-split", action="store_true",
                    help="N > 1: every rank keeps the whole LM head instead of its slice of the vocabulary")
    ap.add_argument("--nvfp4-expand", action="store_true",
                    help="NVFP4 experts on the de-quantising GEMM (W4A16) instead of the native W4A4 path")
    ap.add_argument("--profile-range", action="store_true",
                    help="after the timed region, replay one decode step between cudaProfilerStart/Stop "
                         "(for a profiler started with --profile-from-start off)")
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the model (result marked invalid)")
    a = ap.parse_args(argv)
    if a.impl == "reference":
        return reference_arm()

    import torch

    from legion_b200.config import PRESETS
    from legion_b200.engine.lm import EngineConfig, LmEngine
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    from legion_b200.loaders.tokenizer import ByteTokenizer
    from legion_b200.models.decoder import Decoder
    from legion_b200.models.weights import Shard
    from legion_b200.ops import sm100
    from legion_b200.parallel import dist as pdist

    rank, local_rank, world = pdist.env_world()
    assert world == a.gpus or (a.gpus == 1 and world == 1), f"--gpus {a.gpus} but WORLD_SIZE={world}"
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    spec = CONFIGS[a.config]
    cfg = PRESETS[spec["model"]]()
    if a.layers:
        cfg.n_layer = a.layers
        cfg.layer_kinds = cfg.layer_kinds[:a.layers]
    W, K, L = max(3, a.warmup), a.steps, a.prompt_len or spec["prompt_len"]
    grid = [int(u) for u in a.grid.split(",") if u.strip()]
    all_users = sorted(set(grid + [a.users]))
    U_max = max(all_users)
    nvfp4, fp8 = spec["weights"] == "nvfp4", spec["weights"] == "fp8"
    ep = world > 1 and cfg.n_expert > 0 and (a.moe == "ep" or (a.moe == "auto" and (world >= 4 or nvfp4 or fp8)))
    pctx = pdist.init_from_env("cuda", comm=a.comm, max_rows=8192, hidden=cfg.hidden, expert_parallel=ep)
    shard = Shard(cfg, rank, world, expert_parallel=ep,
                  shared_whole=ep and (nvfp4 or fp8) and not a.no_fold and cfg.shared_ff == cfg.expert_ff) if world > 1 else None
    t0 = time.time()
    weights = build_model(a, cfg, dev, pctx, shard, spec["weights"])
    load_s = time.time() - t0
    tok = ByteTokenizer(cfg.vocab)
    g = torch.Generator().manual_seed(1234)
    extra = {"weights_init_s": round(load_s, 1)}
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def drive_prefill(eng, n_seqs):
        """Steps the engine on this thread until every sequence decodes; returns the device time in ms."""
        eng._drain(block=False)
        pdist.barrier(); torch.cuda.synchronize()
        ev0.record()
        guard = 0
        while True:
            eng._admit()
            if eng.running and all(s.phase == "decode" for s in eng.running) and len(eng.waiting) == 0:
                break
            eng.step()
            guard += 1
            assert guard < 10000
        ev1.record()
        torch.cuda.synchronize()
        assert len(eng.running) == n_seqs
        return pdist.all_reduce_max(ev0.elapsed_time(ev1), dev)

    # ------------------------------------------------------------------ one long prompt: prefill tokens/s
    if a.prefill_len > 0:
        PL = a.prefill_len
        ec = EngineConfig(ctx_size=PL + 64, max_seqs=1, max_batch_tokens=8192, prefill_chunk=8192, block_size=64,
                          prefix_cache=False, device=str(dev), model_name=spec["model"], cuda_graphs=False)
        model = Decoder(cfg, weights, pctx, max_position=ec.ctx_size + 8)
        model.fuse_gdn_in_proj()
        eng = LmEngine(model, tok, ec, start=False)
        times = []
        for rep in range(3):
            prompt = torch.randint(0, cfg.vocab, (PL,), generator=g, dtype=torch.int32).tolist()
            st = eng.generate(GenerateRequest(prompt_tokens=prompt, request_id=f"p{rep}",
                                              sampling=SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)))
            times.append(drive_prefill(eng, 1))
            st.cancel()
            eng._handle_cancels()
            for _ in range(2):
                eng.step()
            assert not eng.running
        ms = statistics.median(times[1:]) if len(times) > 1 else times[0]     # the first pass also sizes workspaces
        extra["prefill_32k"] = {"prompt_len": PL, "tok_s": round(PL / (ms / 1000.0), 1), "ms": round(ms, 1),
                                "ms_all": [round(t, 1) for t in times], "chunk": 8192}
        del eng, model
        import gc
        gc.collect()
        torch.cuda.empty_cache()

    # ------------------------------------------------------------------ decode rows
    gen_budget = (len(all_users) + 1) * ((W + K) * (a.repeats + 2) + 64) + 2 * U_max
    ec = EngineConfig(ctx_size=L + gen_budget + 64, max_seqs=U_max, max_batch_tokens=8192, prefill_chunk=8192,
                      block_size=64, prefix_cache=False, device=str(dev), model_name=spec["model"])
    model = Decoder(cfg, weights, pctx, max_position=ec.ctx_size + 8)
    model.fuse_gdn_in_proj()
    model.fuse_mla_in_proj()
    model.absorb_mla_q()            # decode steps: no per-head absorb GEMM (the folded weight is three times q_b)
    head_split = (not a.no_head_split) and model.split_head()
    eng = LmEngine(model, tok, ec, start=False)
    graphs = eng._graphs
    assert graphs is not None, "decode steps must run from captured CUDA graphs"
    rows = {}
    headline = None
    clk = None
    for U in all_users:
        prompts = torch.randint(0, cfg.vocab, (U, L), generator=g, dtype=torch.int32).pin_memory()
        streams = [eng.generate(GenerateRequest(prompt_tokens=prompts[u].tolist(), request_id=f"u{U}_{u}",
                                                sampling=SamplingParams(temperature=0.0, max_tokens=gen_budget,
                                                                        ignore_eos=True))) for u in range(U)]
        prefill_ms = drive_prefill(eng, U)
        for _ in range(W):
            eng.step()
        is_head = U == a.users
        row = {"users": U, "prompt_len": L, "prefill_ms": round(prefill_ms, 1)}
        if is_head:
            # ---- e2e through the engine's step (pinned H2D of inputs + D2H of picks every step)
            pdist.barrier(); torch.cuda.synchronize()
            h2d0, d2h0, rep0 = graphs.h2d_bytes, graphs.d2h_bytes, graphs.replays
            host0 = dict(eng._stats.host_ms)
            t_e2e0 = time.perf_counter()
            for _ in range(K):
                eng.step()
            torch.cuda.synchronize()
            e2e_s = pdist.all_reduce_max(time.perf_counter() - t_e2e0, dev)
            replays = graphs.replays - rep0
            assert replays == K, "decode steps did not run through the captured graph"
            row["e2e"] = {"value": round(U * K / e2e_s, 2), "unit": "tok/s",
                          "h2d_bytes_per_step": int((graphs.h2d_bytes - h2d0) / replays),
                          "d2h_bytes_per_step": int((graphs.d2h_bytes - d2h0) / replays), "steps": K,
                          # host time per step by phase (forward = pack + upload + graph launch + wait for the picks)
                          "host_ms_per_step": {k: round((v - host0.get(k, 0.0)) / K, 4)
                                               for k, v in eng._stats.host_ms.items()}}
        assert len(eng.running) == U and all(not s.finished for s in eng.running), \
            "a sequence finished before the timed region: the step no longer carries the full batch"
        entry = graphs.entries[graphs.bucket(U)]
        if is_head:
            # kernels per step: counted once with an eager run of the same step on the same inputs
            sm100.LAUNCHES["n"] = 0
            eng.model.forward(entry.batch, eng.kv, eng.states)
            sm100.argmax(torch.zeros(U, cfg.vocab, device=dev))
            torch.cuda.synchronize()
            row["launches_per_step"] = sm100.LAUNCHES["n"]
        for _ in range(W):
            entry.graph.replay()
        clocks = ClockSampler(local_rank) if is_head else None
        if clocks:
            clocks.start()
        reps = []
        for _ in range(max(1, a.repeats)):
            pdist.barrier(); torch.cuda.synchronize()
            ev0.record()
            for _ in range(K):
                entry.graph.replay()
            ev1.record()
            torch.cuda.synchronize()
            pdist.barrier()
            reps.append(pdist.all_reduce_max(ev0.elapsed_time(ev1), dev) / K)
        if clocks:
            clk = clocks.stop()
        if a.profile_range and is_head:
            torch.cuda.profiler.start()
            entry.graph.replay()
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        ms = statistics.median(reps)
        row.update({"ms_per_step": round(ms, 4), "tok_s": round(U * 1000.0 / ms, 2),
                    "ms_min": round(min(reps), 4), "ms_max": round(max(reps), 4), "repeats": len(reps), "steps": K})
        rows[U] = row
        if is_head:
            headline = row
        for s in streams:
            s.cancel()
        eng._handle_cancels()
        for _ in range(2):
            eng.step()
        assert not eng.running, "cancelled sequences are still running"
    status = sm100.Workspace.get(dev).check()
    comm_status = int(pctx.symm.status.item()) if pctx.symm is not None else 0

    par = "single GPU" if world == 1 else (f"tp{world}" + ("+ep(experts whole per rank, tokens mirrored)" if ep else ""))
    extra.update({"decode": {str(u): rows[u] for u in all_users}, "kernel_status_word": status,
                  "comm_status_word": comm_status, "lm_head": "split by vocabulary rows" if head_split else "whole per rank", "launches_per_step": headline.get("launches_per_step"),
                  "shared_expert": ("stacked behind the routed experts (one slot of the grouped GEMMs)"
                                    if (nvfp4 and world == 1 and not a.no_fold and cfg.shared_ff) else
                                    ("whole on rank (layer % world), stacked behind that rank's routed experts"
                                     if (shard is not None and shard.shared_whole) else "dense FFN")),
                  "region": f"median of {len(reps)} regions of {K} steps; min / max per row"})
    out = {
        "metric": f"decode tok/s @{a.users} users ({L}-token prompts), device-timed",
        "value": headline["tok_s"], "unit": "tok/s", "n_gpus": a.gpus, "steps": K, "warmup": W,
        "ms_per_step": headline["ms_per_step"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": spec["dtype"], "data": "synthetic",
        "config": {"model": spec["model"] + ("" if not a.layers else f"-TRUNCATED-{a.layers}L-INVALID"),
                   "baseline_config": a.config, "global_batch": a.users, "seq_len": L, "parallelism": par,
                   "users": a.users, "comm": a.comm if a.gpus > 1 else "none",
                   "l2": "inputs larger than L2 (each step streams several GB of weights, recurrent state and KV)",
                   "page": 64, "weights": spec["weights"]},
        "clocks": clk,
        "e2e": headline.get("e2e"),
        "gpu_launches": int(headline.get("launches_per_step", 0) * K * max(1, a.repeats)),
        "extra": extra,
    }
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch.distributed as dist
        eng.release_graphs()
        torch.cuda.synchronize()
        dist.barrier()
        # the JSON line is out; a teardown that blocks must not hold the launcher
        guard = threading.Timer(20.0, lambda: os._exit(0))
        guard.daemon = True
        guard.start()
        dist.destroy_process_group()
        guard.cancel()
    return 0


if __name__ == "__main__":
    sys.exit(main())
