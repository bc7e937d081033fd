"""``legion`` command line: ``serve | run | bench | chat | top | gguf | st | info | tokenize | ep-place | completions``
plus ``kernel-bench`` (the per-kernel developer benchmarks). Same verbs and flag names as the reference CLI
(``src/cli/mod.rs:83-216``, flags ``docs/serving.md:20-414``); flags that only select between the reference's
ggml-compatible kernel variants have no meaning here and are not present.

    python -m legion_b200 serve --model random:tiny-hybrid-moe --port 8090
    python -m legion_b200 run --model model.gguf -p "Hello" -n 64
"""
from __future__ import annotations

import argparse
import json
import logging
import os
import sys
import time
from typing import List, Optional


def _add_engine_args(ap: argparse.ArgumentParser):
    g = ap.add_argument_group("model")
    g.add_argument("--model", "-m", help="a .gguf file, an HF checkpoint directory or random:<preset>")
    g.add_argument("--hfmodel", help="HF checkpoint directory (same as --model for a directory)")
    g.add_argument("--device", default=None, help="cpu | cuda | cuda:N (default: cuda when available)")
    g.add_argument("--alias", default=None, help="model id reported by /v1/models")
    g = ap.add_argument_group("engine")
    g.add_argument("--ctx-size", type=int, default=8192)
    g.add_argument("--max-seqs", type=int, default=None,
                   help="sequences in flight (default by device memory: 16 on 70 GB and more, fewer on smaller parts)")
    g.add_argument("--max-batch-tokens", type=int, default=None)
    g.add_argument("--prefill-chunk", type=int, default=None)
    g.add_argument("--kv-cache-tokens", type=lambda v: -1 if v == "auto" else int(v), default=None,
                   help="tokens of KV cache; 'auto' = as many as fit the GPU beside the weights (memory plan); default "
                        "max-seqs x ctx-size")
    g.add_argument("--gpu-memory-utilization", type=float, default=None,
                   help="share of the device's memory the memory plan may fill")
    g.add_argument("--kv-block", type=int, default=None, help="tokens per KV block (64 on GPU, 16 on CPU)")
    g.add_argument("--no-prefix-cache", action="store_true")
    g.add_argument("--kv-rings", action="store_true",
                   help="sliding-window layers keep window + one step of K / V per sequence in a ring of blocks instead "
                        "of pages for the whole context (prompts then resume from the prefix cache at state snapshots only)")
    g.add_argument("--prefix-cache-states", type=int, default=8)
    g.add_argument("--prefix-cache-interval", type=int, default=0)
    g.add_argument("--max-waiting", type=int, default=1024)
    g.add_argument("--default-max-tokens", type=int, default=4096)
    g.add_argument("--scheduling-policy", choices=["fcfs", "priority"], default="fcfs")
    g.add_argument("--fair-share", action="store_true")
    g.add_argument("--kv-admission", choices=["reserve", "on-demand"], default="reserve")
    g.add_argument("--kv-swap-gib", type=float, default=0.0,
                   help="pinned host memory for the KV / state of preempted sequences (0: recompute them)")
    g.add_argument("--prefix-cache-host-gib", type=float, default=0.0,
                   help="pinned host memory that keeps the contents of prefix-cache blocks evicted from HBM; a later "
                        "prompt with that prefix copies them back instead of recomputing (0: evicted blocks are dropped)")
    g.add_argument("--itl-target", type=float, default=0.0, help="inter-token latency target (ms) for the prompt budget")
    g.add_argument("--ttft-target", type=float, default=0.0)
    g.add_argument("--deterministic", action="store_true")
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--no-cuda-graphs", action="store_true")
    g.add_argument("--nvtx", action="store_true", help="NVTX range around every eager step")
    g.add_argument("--op-profile", action="store_true",
                   help="time every kernel call between CUDA events (use with --no-cuda-graphs); table at exit of run")
    g = ap.add_argument_group("speculative decoding")
    g.add_argument("--spec", choices=["none", "ngram", "suffix", "mtp", "mtp_ngram", "draft", "eagle3", "dflash"],
                   default="none")
    g.add_argument("--spec-k", type=int, default=4)
    g.add_argument("--spec-max-batch", type=int, default=8)
    g.add_argument("--spec-draft-model", default=None,
                   help="--spec eagle3: the head's checkpoint directory (config.json + safetensors); --spec draft: the "
                        "draft model (same vocabulary as the target)")
    g.add_argument("--spec-p-min", type=float, default=0.5,
                   help="--spec-policy adaptive: a sequence drafts as deep as its last draft keeps this acceptance probability")
    g.add_argument("--spec-policy", choices=["fixed", "cost", "adaptive"], default="fixed",
                   help="cost: pick the draft depth per step from the measured acceptance rate and batch size; adaptive: "
                        "per-sequence acceptance along the chain plus measured verify / draft step costs")
    g.add_argument("--no-even-chunks", action="store_true", help="full prompt chunks plus a short tail")
    g = ap.add_argument_group("parallelism")
    g.add_argument("--tp", type=int, default=1, help="tensor-parallel ranks (one process per GPU, spawned by serve)")
    g.add_argument("--gpus", type=int, default=None, help="alias of --tp on a single node")
    g.add_argument("--tp-moe-ep", action="store_true", help="shard whole experts over the ranks instead of their rows")
    g.add_argument("--tp-comm", choices=["fused", "nccl"], default="fused")
    g.add_argument("--dp-attention", action="store_true",
                   help="with --tp N: every rank holds attention whole and runs it for its own sequences; routed "
                        "experts are split over the ranks and tokens travel to them inside each MoE layer")
    g.add_argument("--ep-capacity", type=float, default=0.0,
                   help="--dp-attention: receive room per rank as a multiple of its own routed pairs (0 = worst case)")
    g.add_argument("--tp-replicas", type=int, default=1, help="data-parallel engine replicas")
    g.add_argument("--tp-gemm-tail", action="store_true",
                   help="run o-proj / down-proj and their all-reduce as one kernel (fused communicator)")
    g.add_argument("--pp", type=int, default=1, help="pipeline stages (layers split over the GPUs, one process each)")
    g.add_argument("--layer-split", default=None, help="layers per pipeline stage, e.g. 7,7,7,7,7,7,7,6")
    g.add_argument("--split-last-extra", type=int, default=0, help="layers' worth of room kept free on the last stage")
    g.add_argument("--pipeline-micro", type=int, default=2048, help="tokens per micro-chunk of a pipelined prompt")
    g.add_argument("--pipeline-groups", type=int, default=0,
                   help="--pp: groups a decode step's sequences travel the stages in, one behind the other (0 = one per "
                        "stage)")
    g.add_argument("--experts", choices=["auto", "device", "host", "cache", "ssd"], default="auto")
    g.add_argument("--expert-cache-gib", type=float, default=0.0)
    g.add_argument("--expert-dir", default=None, help="--experts ssd: directory of the per-layer expert files")
    g.add_argument("--expert-ram-gib", type=float, default=8.0,
                   help="--experts ssd: host memory for recently used experts between the files and the HBM slots")
    g.add_argument("--mmproj", default=None, help="vision tower: a clip mmproj GGUF (qwen3vl_merger projector)")
    g.add_argument("--no-mmproj", action="store_true", help="do not load the vision tower a checkpoint directory ships")
    g.add_argument("--image-max-tokens", type=int, default=0, help="most rows one image may take (0 = the tower's limit)")
    g.add_argument("--image-cache-mib", type=int, default=256, help="encoded image rows kept by image hash")
    g.add_argument("--numa", choices=["auto", "off"], default="auto",
                   help="auto: restrict each rank's host threads to the CPUs of its GPU's NUMA node")
    g.add_argument("--load-threads", type=int, default=8,
                   help="threads of positional reads that fetch a checkpoint layer ahead of the loader (0 = memory map only)")
    g.add_argument("--expert-weights", choices=["bf16", "nvfp4", "fp8"], default="bf16",
                   help="nvfp4: keep the routed experts in 4 bits in HBM (expanded inside the grouped GEMM); "
                        "fp8: block-scaled e4m3 experts on the FP8 tensor-core path")
    g.add_argument("--weights", choices=["auto", "bf16", "fp8"], default="auto",
                   help="fp8: keep all projection weights in block-scaled e4m3 (128 x 128 scales) in HBM and run them "
                        "on the FP8 tensor-core path; auto: fp8 for checkpoints shipped in block-scaled FP8 (the "
                        "re-encoding of their expanded blocks reproduces the shipped bytes), bf16 otherwise")
    g = ap.add_argument_group("sampling defaults")
    g.add_argument("--temp", type=float, default=None)
    g.add_argument("--top-p", type=float, default=None)
    g.add_argument("--top-k", type=int, default=None)
    g.add_argument("--min-p", type=float, default=None)
    g.add_argument("--tool-format", choices=["hermes", "qwen3_coder", "glm", "gemma4"], default="hermes")


def build_engine_from_args(a, start: bool = True):
    import torch

    from ..engine.lm import EngineConfig, LmEngine
    from ..engine.mock import MockEngine
    from ..loaders.model import load_model
    from ..models.decoder import Decoder
    from ..parallel import dist as pdist

    path = a.model or a.hfmodel
    if not path:
        return MockEngine(a.alias or "mock")
    device = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    rank, local_rank, world = pdist.env_world()
    if world > 1 and device.startswith("cuda"):
        device = f"cuda:{local_rank}"
    on_gpu = device.startswith("cuda")
    from ..hw.defaults import engine_defaults
    hd = engine_defaults(device)          # sizes the command line left open come from what the device reports
    logging.getLogger("legion").info("hardware profile %s: chunk %d, page %d, %d sequences", hd.profile,
                                     a.prefill_chunk or hd.prefill_chunk, a.kv_block or hd.kv_block,
                                     a.max_seqs or hd.max_seqs)
    ec = EngineConfig(
        ctx_size=a.ctx_size, max_seqs=a.max_seqs or hd.max_seqs,
        max_batch_tokens=a.max_batch_tokens or hd.max_batch_tokens,
        prefill_chunk=a.prefill_chunk or hd.prefill_chunk, block_size=a.kv_block or hd.kv_block,
        kv_cache_tokens=a.kv_cache_tokens,
        gpu_memory_utilization=getattr(a, "gpu_memory_utilization", None) or hd.gpu_memory_utilization or 0.92,
        kv_fit_check=True, prefix_cache=not a.no_prefix_cache, kv_rings=getattr(a, "kv_rings", False),
        prefix_cache_states=a.prefix_cache_states, prefix_cache_interval=a.prefix_cache_interval,
        max_waiting=a.max_waiting, default_max_tokens=a.default_max_tokens, scheduling_policy=a.scheduling_policy,
        fair_share=a.fair_share, kv_admission=a.kv_admission, spec=a.spec, spec_k=a.spec_k, spec_draft_model=getattr(a, "spec_draft_model", None),
        spec_max_batch=a.spec_max_batch, deterministic=a.deterministic, device=device, seed=a.seed,
        cuda_graphs=not a.no_cuda_graphs, model_name=a.alias or os.path.basename(path.rstrip("/")),
        tool_format=a.tool_format, itl_target_ms=a.itl_target, ttft_target_ms=a.ttft_target,
        nvtx=getattr(a, "nvtx", False), kv_swap_gib=getattr(a, "kv_swap_gib", 0.0),
        prefix_host_gib=getattr(a, "prefix_cache_host_gib", 0.0), spec_policy=getattr(a, "spec_policy", "fixed"), spec_p_min=getattr(a, "spec_p_min", 0.5), even_chunks=not getattr(a, "no_even_chunks", False))
    pctx = None
    if world > 1 and getattr(a, "pp", 1) > 1:
        # pipeline stages: every rank loads only its layers, the residual travels by send / recv
        import torch.distributed as dist
        from ..config import PRESETS
        from ..parallel.pipeline import PipeStage
        pdist.init_from_env(device, comm="nccl")
        n_layer = PRESETS[path.split(":", 1)[1]]().n_layer if path.startswith("random:") else None
        if n_layer is None:
            n_layer = load_model(path, "cpu", keep_layers=lambda il: False)[0].n_layer
        split = [int(x) for x in a.layer_split.split(",")] if a.layer_split else None
        pipe = PipeStage(rank, world, dist.group.WORLD, n_layer, split, a.pipeline_micro, a.split_last_extra,
                         decode_groups=getattr(a, "pipeline_groups", 0) or world)
        cfg, w, tok, info = load_model(path, device, seed=a.seed, keep_layers=pipe.owns)
        model = Decoder(cfg, w, None, max_position=ec.ctx_size + 8, pipe=pipe)
        return LmEngine(model, tok, ec, start=start)
    if world > 1 and getattr(a, "dp_attention", False):
        import torch.distributed as dist
        from ..parallel.context import DpEpCtx
        pdist.init_from_env(device, comm="nccl")
        cfg, w, tok, info = load_model(path, device, rank=rank, world=world, seed=a.seed, dp_attention=True)
        disp = None
        if on_gpu and cfg.n_expert:
            from ..parallel.ep import EpDispatcher
            disp = EpDispatcher(dist.group.WORLD, rank, world, torch.device(device), cfg.n_expert, cfg.top_k, cfg.hidden,
                                cfg.expert_ff, ec.max_batch_tokens, a.ep_capacity or None)
        model = Decoder(cfg, w, DpEpCtx(rank, world, dist.group.WORLD, disp), max_position=ec.ctx_size + 8)
        return LmEngine(model, tok, ec, start=start)
    if world > 1:
        from ..config import PRESETS  # noqa: F401
        pctx = pdist.init_from_env(device, comm="nccl", expert_parallel=a.tp_moe_ep)   # symmetric memory is attached
        # below, once the model's hidden size is known
    if on_gpu and getattr(a, "numa", "auto") == "auto":
        from ..hw.numa import bind_to_gpu
        placed = bind_to_gpu(torch.device(device).index or 0)
        if placed["bound"]:
            logging.getLogger("legion").info("rank %d: host threads on NUMA node %s (%d CPUs) next to GPU %s", rank,
                                             placed["node"], len(placed["cpus"]), placed["bus_id"])
    # block-quantised checkpoints stay in their shipped encoding on a GPU (no bf16 copy on the way in) unless the
    # experts are offloaded (the host tiers hold plain tensors) or bf16 weights were asked for
    keep_q = (on_gpu and getattr(a, "weights", "auto") != "bf16" and a.experts not in ("cache", "host", "ssd"))
    cfg, w, tok, info = load_model(path, device, rank=rank, world=world, expert_parallel=a.tp_moe_ep, seed=a.seed,
                                   keep_quant=keep_q, read_threads=getattr(a, "load_threads", 0))
    if pctx is not None and pctx.symm is None and a.tp_comm == "fused" and on_gpu:
        from ..parallel.symm import SymmComm
        import torch.distributed as dist
        pctx.symm = SymmComm(dist.group.WORLD, rank, world, torch.device(device), ec.max_batch_tokens, cfg.hidden)
        pctx.comm = "fused"
        pctx.gemm_tail = bool(getattr(a, "tp_gemm_tail", False))
    model = Decoder(cfg, w, pctx, max_position=ec.ctx_size + 8)
    if on_gpu:
        model.fuse_gdn_in_proj()
        model.split_head()       # several ranks with the fused communicator: each keeps its slice of the vocabulary
    if getattr(a, "expert_weights", "bf16") == "nvfp4" and on_gpu and cfg.n_expert:
        if pctx.world == 1 and a.experts not in ("cache", "host", "ssd"):
            model.fold_shared_experts()      # the shared expert rides in the grouped GEMMs of decode steps
        saved = model.quantize_experts_nvfp4()
        logging.getLogger("legion").info("routed experts re-encoded to NVFP4: %.1f GiB of HBM saved", saved / 2 ** 30)
    wmode = getattr(a, "weights", "auto")
    if wmode == "auto":
        wmode = "fp8" if info.get("quant_method") == "fp8_block" else "bf16"
    if on_gpu and (wmode == "fp8" or getattr(a, "expert_weights", "bf16") == "fp8"):
        saved = model.quantize_weights_fp8(experts_only=wmode != "fp8")
        logging.getLogger("legion").info("weights re-encoded to block-scaled FP8: %.1f GiB of HBM saved", saved / 2 ** 30)
    if a.experts in ("cache", "host", "ssd") and cfg.n_expert:
        from ..residency.experts import slots_for_budget
        slots = cfg.top_k * ec.max_seqs if a.experts == "host" else slots_for_budget(cfg, a.expert_cache_gib or 8.0)
        if a.experts == "ssd":
            if not a.expert_dir:
                raise SystemExit("--experts ssd needs --expert-dir")
            model.offload_experts(max(slots, cfg.top_k), ssd_dir=a.expert_dir,
                                  ram_experts=slots_for_budget(cfg, a.expert_ram_gib))
        else:
            model.offload_experts(max(slots, cfg.top_k))
    eng = LmEngine(model, tok, ec, start=start)
    _attach_vision(a, eng, path, device)
    logging.getLogger("legion").info("loaded %s: %s, %d layers, %.2fB parameters on %s", path, cfg.arch, cfg.n_layer,
                                     sum((t.numel() if isinstance(t, torch.Tensor) else t.codes.numel() * 2 if hasattr(t, "codes")
                                          else t.data.numel()) for t in w.values() if t is not None) / 1e9, device)
    if a.tp_replicas > 1:
        from ..engine.replicas import ReplicaEngine
        return ReplicaEngine([eng] + [LmEngine(model, tok, ec) for _ in range(a.tp_replicas - 1)])
    return eng


def _attach_vision(a, eng, path: str, device) -> None:
    """``--mmproj FILE`` (a ``clip`` mmproj GGUF) or the tower a Hugging Face checkpoint directory ships."""
    import torch
    from ..vision import VisionRuntime
    mm = getattr(a, "mmproj", None)
    dt = torch.bfloat16 if str(device).startswith("cuda") else torch.float32
    got = None
    if mm:
        from ..loaders.vision import load_mmproj
        got = load_mmproj(mm, device, dt)
    elif os.path.isdir(path) and os.path.exists(os.path.join(path, "config.json")) and not getattr(a, "no_mmproj", False):
        from ..loaders.vision import load_vision_hf
        try:
            got = load_vision_hf(path, device, dt)
        except Exception as e:      # a checkpoint whose tower cannot be read still serves text
            logging.getLogger("legion").warning("vision tower of %s not loaded: %s", path, e)
            return
    if got is None:
        return
    tower, hp = got
    if getattr(a, "image_max_tokens", 0):
        hp.image_max_pixels = hp.factor * hp.factor * int(a.image_max_tokens)
    eng.attach_vision(VisionRuntime(tower, hp, cache_bytes=int(getattr(a, "image_cache_mib", 256)) << 20))
    logging.getLogger("legion").info("vision tower: %d blocks of width %d, up to %d tokens per image", tower.cfg.depth,
                                     tower.cfg.hidden, hp.max_image_tokens())


def sampling_defaults(a) -> dict:
    return {k: v for k, v in (("temperature", a.temp), ("top_p", a.top_p), ("top_k", a.top_k), ("min_p", a.min_p))
            if v is not None}


# ------------------------------------------------------------------------------------------------ commands
def cmd_serve(a):
    from ..server.app import ServerConfig, serve
    tp = max(a.gpus or a.tp, getattr(a, "pp", 1))
    if tp > 1 and "RANK" not in os.environ:
        # one process per GPU: re-launch this command under torch.distributed.run; rank 0 serves HTTP
        import subprocess
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={tp}",
               "--master-addr", "127.0.0.1", "--master-port", str(a.master_port), "-m", "legion_b200"] + sys.argv[1:]
        return subprocess.call(cmd)
    logging.basicConfig(level=getattr(logging, a.log_level.upper()), format="%(asctime)s %(levelname)s %(name)s: %(message)s")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    eng = build_engine_from_args(a, start=world == 1)
    if world > 1:
        from ..parallel import spmd
        spmd.attach(eng, int(os.environ.get("RANK", "0")), world)
        eng.start()
    eng.set_warming(True)
    if a.warmup and hasattr(eng, "generate_text") and world == 1:
        for n in (64, 16):
            eng.generate_text(tokens=list(range(1, n + 1)), max_tokens=2, ignore_eos=True)
    eng.set_warming(False)
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        from ..parallel.spmd import follower_wait
        return follower_wait(eng)
    keys = list(a.api_key or [])
    if os.environ.get("LEGION_API_KEY"):
        keys.append(os.environ["LEGION_API_KEY"])
    cfg = ServerConfig(api_keys=keys, max_request_mb=a.max_request_mb, default_max_tokens=a.default_max_tokens,
                       sampling_defaults=sampling_defaults(a), shutdown_timeout_s=a.shutdown_timeout_secs,
                       fair_share=a.fair_share)
    if a.tui:
        from ..server.dashboard import start_tui
        start_tui(eng)
    print(f"legion-b200 listening on http://{a.host}:{a.port}", flush=True)
    serve(eng, a.host, a.port, cfg, a.tls_cert, a.tls_key, a.log_level)
    return 0


def cmd_run(a):
    from ..engine.types import ChatMessage, GenerateRequest, SamplingParams
    if getattr(a, "op_profile", False):
        from ..ops import sm100
        sm100.op_profile(True)
    eng = build_engine_from_args(a)
    sp = SamplingParams(temperature=a.temp if a.temp is not None else 0.0, top_p=a.top_p or 1.0, top_k=a.top_k or 0,
                        min_p=a.min_p or 0.0, max_tokens=a.n_predict, ignore_eos=a.ignore_eos, seed=a.seed)
    images = []
    for fn in getattr(a, "image", None) or []:
        with open(fn, "rb") as f:
            images.append(f.read())
    if a.chat or images:
        content = a.prompt if not images else [{"type": "image"} for _ in images] + [{"type": "text", "text": a.prompt}]
        req = GenerateRequest(messages=[ChatMessage("user", content)], sampling=sp, images=images)
    else:
        req = GenerateRequest(prompt=a.prompt, sampling=sp)
    t0 = time.time()
    n = 0
    usage = None
    for ev in eng.generate(req):
        if ev.kind in ("text", "reasoning"):
            sys.stdout.write(ev.text)
            sys.stdout.flush()
            n += len(ev.token_ids)
        elif ev.kind == "finished":
            usage = ev.usage
        elif ev.kind == "error":
            print(f"\nerror: {ev.error}", file=sys.stderr)
            return 1
    dt = time.time() - t0
    if getattr(a, "op_profile", False):
        from ..ops import sm100
        print("\n\nop                        calls   total ms   mean us   share")
        for name, calls, ms, us, share in sm100.op_profile_report():
            print(f"{name:24s} {calls:6d} {ms:10.3f} {us:9.1f} {share * 100:6.1f}%")
    if usage:
        print(f"\n\n[{usage.prompt_tokens} prompt tokens ({usage.cached_tokens} cached), {usage.completion_tokens} generated, "
              f"prefill {usage.prefill_ms:.0f} ms, decode {usage.decode_ms:.0f} ms, {n / max(dt, 1e-9):.1f} tok/s]",
              file=sys.stderr)
    eng.shutdown()
    return 0


def cmd_chat(a):
    import urllib.request
    history = []
    print("legion chat - empty line to quit")
    while True:
        try:
            line = input("> ").strip()
        except EOFError:
            break
        if not line:
            break
        history.append({"role": "user", "content": line})
        body = json.dumps({"model": "default", "messages": history, "stream": True, "max_tokens": a.n_predict}).encode()
        req = urllib.request.Request(a.url.rstrip("/") + "/v1/chat/completions", data=body,
                                     headers={"content-type": "application/json",
                                              **({"authorization": f"Bearer {a.api_key}"} if a.api_key else {})})
        reply = ""
        with urllib.request.urlopen(req) as r:
            for raw in r:
                raw = raw.decode().strip()
                if not raw.startswith("data: ") or raw == "data: [DONE]":
                    continue
                d = json.loads(raw[6:])
                for c in d.get("choices", []):
                    t = c.get("delta", {}).get("content") or ""
                    reply += t
                    sys.stdout.write(t)
                    sys.stdout.flush()
        print()
        history.append({"role": "assistant", "content": reply})
    return 0


def cmd_bench(a):
    from ..bench.client import run_bench
    return run_bench(a)


def cmd_gguf(a):
    from ..loaders.gguf import GgufFile
    if a.action == "inspect":
        g = GgufFile(a.file)
        print(f"{a.file}: arch={g.arch} tensors={len(g.tensors)} metadata={len(g.metadata)}")
        for k, v in g.metadata.items():
            s = repr(v)
            print(f"  {k} = {s if len(s) < 100 else s[:97] + '...'}")
        if a.tensors:
            for t in g.tensors.values():
                print(f"  {t.name:48s} {t.type_name:6s} {list(t.shape)}")
        return 0
    if a.action == "diff":
        g1, g2 = GgufFile(a.file), GgufFile(a.other)
        rc = 0
        for k in sorted(set(g1.metadata) | set(g2.metadata)):
            if g1.metadata.get(k) != g2.metadata.get(k) and not k.startswith("general."):
                print(f"metadata {k}: {g1.metadata.get(k)!r} != {g2.metadata.get(k)!r}")
                rc = 1
        import numpy as np
        for n in sorted(set(g1.tensors) | set(g2.tensors)):
            if n not in g1.tensors or n not in g2.tensors:
                print(f"tensor {n}: only in {'first' if n in g1.tensors else 'second'}")
                rc = 1
                continue
            x, y = g1.numpy(n), g2.numpy(n)
            if x.shape != y.shape:
                print(f"tensor {n}: shape {x.shape} != {y.shape}")
                rc = 1
            else:
                d = float(np.abs(x.astype(np.float64) - y.astype(np.float64)).max()) if x.size else 0.0
                if d > a.tol:
                    print(f"tensor {n}: max abs diff {d:.3g}")
                    rc = 1
        print("identical" if rc == 0 else "different")
        return rc
    if a.action == "check":
        from ..loaders.gguf_map import load_gguf
        cfg, w, _ = load_gguf(a.file)
        from ..models.weights import weight_shapes
        want = weight_shapes(cfg)
        bad = [k for k, s in want.items() if k not in w or tuple(w[k].shape) != tuple(s)]
        for k in bad:
            print(f"{k}: expected {want[k]}, file has {tuple(w[k].shape) if k in w else 'nothing'}")
        print(f"{cfg.arch}: {len(want) - len(bad)}/{len(want)} tensors ok")
        return 1 if bad else 0
    return 2


def cmd_st(a):
    from ..loaders.safetensors_io import Checkpoint
    ck = Checkpoint(a.path)
    print(f"{a.path}: {len(ck.where)} tensors, quantisation: {ck.quant_method()}")
    if ck.config:
        print(f"  model_type={ck.config.get('model_type')} layers={ck.config.get('num_hidden_layers')}")
    if a.tensors:
        for n in sorted(ck.where):
            dt, shp = ck._open(ck.where[n]).info(n)
            print(f"  {n:72s} {dt:8s} {list(shp)}")
    return 0


def cmd_info(a):
    from ..hw.gpu import system_report
    print(json.dumps(system_report(), indent=1))
    return 0


def cmd_determinism(a):
    """Runs the same prompts on two freshly built engines (and twice on each: cold, then through the prefix cache)
    and compares the generated token ids byte for byte (the reference's ``scripts/determinism.py``)."""
    import torch

    from ..engine.types import GenerateRequest, SamplingParams
    prompts = []
    g = torch.Generator().manual_seed(a.seed)
    for i in range(a.prompts):
        n = int(torch.randint(a.prompt_len // 2, a.prompt_len + 1, (1,), generator=g))
        prompts.append(torch.randint(1, 255, (n,), generator=g).tolist())
    runs = []
    for r in range(2):
        eng = build_engine_from_args(a)
        for rep_ in range(2):
            streams = [eng.generate(GenerateRequest(prompt_tokens=p, sampling=SamplingParams(
                temperature=0.0, max_tokens=a.n_predict, ignore_eos=True))) for p in prompts]
            runs.append([s.collect().token_ids for s in streams])
        eng.shutdown()
    ok = all(r == runs[0] for r in runs[1:])
    for i, r in enumerate(runs[1:], 1):
        diff = sum(1 for x, y in zip(r, runs[0]) if x != y)
        print(f"run {i} vs run 0: {'identical' if diff == 0 else f'{diff} of {len(r)} sequences differ'}")
    print("deterministic" if ok else "NOT deterministic")
    return 0 if ok else 1


def cmd_tokenize(a):
    from ..loaders.model import load_model
    _, _, tok, _ = load_model(a.model, "cpu") if not a.model.startswith("random:") else (None, None, __import__(
        "legion_b200.loaders.tokenizer", fromlist=["ByteTokenizer"]).ByteTokenizer(4096), None)
    ids = tok.encode(a.text, add_special=a.add_special)
    print(json.dumps({"ids": ids, "n": len(ids), "pieces": [tok.decode([i]) for i in ids]} if a.pieces else ids))
    return 0


def cmd_logits(a):
    """Reference logits of a prompt (the role of the reference's ``tools/llama-ref`` dumpers): the prompt runs through
    the model in one pass on the chosen device (``--device cpu`` = the fp32 reference forward), the logits of the
    asked rows go to an ``.npz`` file, and ``--compare`` prints how far another dump is from this one."""
    import numpy as np
    import torch
    eng = build_engine_from_args(a, start=False)
    from ..engine.types import GenerateRequest, SamplingParams
    if a.tokens:
        req = GenerateRequest(prompt_tokens=[int(t) for t in a.tokens.split(",")], sampling=SamplingParams(max_tokens=1))
    else:
        req = GenerateRequest(prompt=a.prompt, sampling=SamplingParams(max_tokens=1))
    seq = eng.prepare(req)
    eng.waiting.push(seq)
    eng._admit()
    n = len(seq.tokens)
    b = eng.build_batch([(seq, 0, n)])
    if a.all_rows:
        b.logit_rows = None
    with torch.no_grad():
        out = eng.model.forward(b, eng.kv, eng.states)
    logits = out.logits.float().cpu().numpy()
    top = logits.argmax(-1)
    if a.out:
        np.savez(a.out, tokens=np.asarray(seq.tokens, dtype=np.int64), logits=logits)
    print(json.dumps({"tokens": n, "rows": int(logits.shape[0]), "argmax_last": int(top[-1]),
                      "max_abs": float(np.abs(logits).max())}))
    if a.compare:
        other = np.load(a.compare)
        if other["logits"].shape != logits.shape or list(other["tokens"]) != list(seq.tokens):
            print("compare: the other dump is of another prompt or row set", file=sys.stderr)
            return 1
        d = np.abs(other["logits"] - logits)
        agree = float((other["logits"].argmax(-1) == top).mean())
        print(json.dumps({"max_abs_diff": float(d.max()), "mean_abs_diff": float(d.mean()), "argmax_agreement": agree}))
    return 0


def cmd_ep_place(a):
    from ..parallel.ep_place import place_from_record
    plan = place_from_record(a.record, a.ranks)
    json.dump(plan, open(a.out, "w") if a.out else sys.stdout, indent=1)
    return 0


def cmd_completions(a):
    subs = ["serve", "run", "bench", "chat", "top", "gguf", "st", "info", "tokenize", "logits", "ep-place", "completions",
            "kernel-bench", "comm-bench"]
    if a.shell == "bash":
        print("complete -W '" + " ".join(subs) + "' legion")
    else:
        print("#compdef legion\n_arguments '1: :(" + " ".join(subs) + ")'")
    return 0


def cmd_top(a):
    from ..server.dashboard import run_top
    return run_top(a.url, a.api_key, a.interval, a.once)


def cmd_kernel_bench(a):
    from ..bench.kernels import main as kmain
    argv = ["--only", a.only] + (["--json", a.json] if a.json else [])
    return kmain(argv)


def cmd_comm_bench(a):
    """One process per GPU under ``torch.distributed.run`` (the communication kernels need their peers)."""
    import subprocess
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(a.gpus),
           "--master-addr", "127.0.0.1", "--master-port", str(a.port), "-m", "legion_b200.bench.comm",
           "--hidden", str(a.hidden), "--rows", a.rows, "--iters", str(a.iters)]
    if a.json:
        cmd += ["--json", a.json]
    return subprocess.call(cmd)


def make_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="legion", description="legion-b200: a Blackwell-native MoE inference engine")
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("serve", help="serve the OpenAI / Anthropic compatible HTTP API")
    _add_engine_args(s)
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--port", type=int, default=8090)
    s.add_argument("--api-key", action="append")
    s.add_argument("--max-request-mb", type=int, default=64)
    s.add_argument("--shutdown-timeout-secs", type=float, default=30.0)
    s.add_argument("--tls-cert")
    s.add_argument("--tls-key")
    s.add_argument("--tui", action="store_true")
    s.add_argument("--no-warmup", dest="warmup", action="store_false")
    s.add_argument("--log-level", default="info")
    s.add_argument("--master-port", type=int, default=29533)
    s.set_defaults(fn=cmd_serve)
    s = sub.add_parser("run", help="generate once and print the text")
    _add_engine_args(s)
    s.add_argument("--prompt", "-p", required=True)
    s.add_argument("--n-predict", "-n", type=int, default=128)
    s.add_argument("--chat", action="store_true", help="wrap the prompt in the chat template")
    s.add_argument("--image", action="append", help="image file shown before the prompt (repeatable; needs a vision tower)")
    s.add_argument("--ignore-eos", action="store_true")
    s.set_defaults(fn=cmd_run)
    s = sub.add_parser("chat", help="terminal chat against a running server")
    s.add_argument("--url", default="http://127.0.0.1:8090")
    s.add_argument("--api-key")
    s.add_argument("--n-predict", "-n", type=int, default=1024)
    s.set_defaults(fn=cmd_chat)
    s = sub.add_parser("bench", help="benchmark client: bench | chats | prefill | mixed | bandwidth")
    s.add_argument("workload", nargs="?", default="bench", choices=["bench", "chats", "prefill", "mixed", "bandwidth"])
    s.add_argument("--url", default="http://127.0.0.1:8090")
    s.add_argument("--api-key")
    s.add_argument("--api", choices=["openai", "anthropic"], default="openai")
    s.add_argument("--concurrency", default="1,4,16")
    s.add_argument("--prompt-tokens", type=int, default=512)
    s.add_argument("--max-tokens", type=int, default=256)
    s.add_argument("--prefill-sizes", default="8192,32768")
    s.add_argument("--rounds", type=int, default=1)
    s.add_argument("--save")
    s.set_defaults(fn=cmd_bench)
    s = sub.add_parser("top", help="live view of a running server's /v1/stats")
    s.add_argument("--url", default="http://127.0.0.1:8090")
    s.add_argument("--api-key")
    s.add_argument("--interval", type=float, default=1.0)
    s.add_argument("--once", action="store_true")
    s.set_defaults(fn=cmd_top)
    s = sub.add_parser("gguf", help="inspect | diff | check a GGUF file")
    s.add_argument("action", choices=["inspect", "diff", "check"])
    s.add_argument("file")
    s.add_argument("other", nargs="?")
    s.add_argument("--tensors", action="store_true")
    s.add_argument("--tol", type=float, default=0.0)
    s.set_defaults(fn=cmd_gguf)
    s = sub.add_parser("st", help="inspect a safetensors checkpoint")
    s.add_argument("action", choices=["inspect"])
    s.add_argument("path")
    s.add_argument("--tensors", action="store_true")
    s.set_defaults(fn=cmd_st)
    s = sub.add_parser("info", help="hardware report: GPUs, NVLink, measured rooflines")
    s.set_defaults(fn=cmd_info)
    s = sub.add_parser("determinism", help="byte-compare the tokens of repeated runs (fresh engines, prefix-cache reuse)")
    _add_engine_args(s)
    s.add_argument("--prompts", type=int, default=4)
    s.add_argument("--prompt-len", type=int, default=96)
    s.add_argument("--n-predict", "-n", type=int, default=16)
    s.set_defaults(fn=cmd_determinism)
    s = sub.add_parser("logits", help="dump (and compare) the logits of a prompt: the reference-logit tool")
    _add_engine_args(s)
    s.add_argument("--prompt", "-p", default="")
    s.add_argument("--tokens", default=None, help="comma-separated token ids instead of --prompt")
    s.add_argument("--all-rows", action="store_true", help="logits of every prompt position, not only the last")
    s.add_argument("--out", default=None, help=".npz file to write (tokens, logits)")
    s.add_argument("--compare", default=None, help=".npz dump to compare with")
    s.set_defaults(fn=cmd_logits)
    s = sub.add_parser("tokenize", help="tokenise text with a model's tokenizer")
    s.add_argument("--model", "-m", required=True)
    s.add_argument("text")
    s.add_argument("--add-special", action="store_true")
    s.add_argument("--pieces", action="store_true")
    s.set_defaults(fn=cmd_tokenize)
    s = sub.add_parser("ep-place", help="co-activation aware expert placement from a route record")
    s.add_argument("record")
    s.add_argument("--ranks", type=int, default=8)
    s.add_argument("--out")
    s.set_defaults(fn=cmd_ep_place)
    s = sub.add_parser("completions", help="shell completion script")
    s.add_argument("shell", choices=["bash", "zsh"])
    s.set_defaults(fn=cmd_completions)
    s = sub.add_parser("kernel-bench", help="device-timed micro-benchmarks of the sm_100a kernels")
    s.add_argument("--only", default="gemm,moe,decode_attn,prefill_attn")
    s.add_argument("--json")
    s.set_defaults(fn=cmd_kernel_bench)
    s = sub.add_parser("comm-bench", help="device-timed fused all-reduce / all-gather kernels against NCCL")
    s.add_argument("--gpus", type=int, default=2)
    s.add_argument("--hidden", type=int, default=2048)
    s.add_argument("--rows", default="16,64,2048")
    s.add_argument("--iters", type=int, default=20)
    s.add_argument("--port", type=int, default=29533)
    s.add_argument("--json")
    s.set_defaults(fn=cmd_comm_bench)
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    a = make_parser().parse_args(argv)
    return int(a.fn(a) or 0)


if __name__ == "__main__":
    sys.exit(main())
