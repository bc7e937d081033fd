"""The engine on a GPU: kernels + scheduler + CUDA-graph decode agree with the fp32 CPU engine."""
import pytest
import torch

from legion_b200.config import PRESETS, ModelConfig, tiny_hybrid_moe
from legion_b200.engine.lm import EngineConfig, build_engine
from legion_b200.models.weights import random_weights

pytestmark = pytest.mark.gpu


def _cfgs():
    return [
        ModelConfig(arch="qwen3moe", n_layer=2, hidden=256, vocab=1024, n_head=4, n_kv_head=2, head_dim=64,
                    n_expert=8, top_k=2, expert_ff=128),
        tiny_hybrid_moe(),
        ModelConfig(arch="qwen3", n_layer=2, hidden=256, vocab=1024, n_head=4, n_kv_head=2, head_dim=128, dense_ff=512),
        # latent attention with the 512 + 64 cache row the tcgen05 kernel implements, MoE with grouped sigmoid routing
        ModelConfig(arch="deepseek_v3", n_layer=3, hidden=256, vocab=1024, n_head=16, n_kv_head=16, head_dim=128,
                    q_lora=96, kv_lora=512, qk_nope_dim=64, qk_rope_dim=64, v_head_dim=64, qk_norm=False,
                    dense_ff=384, first_dense_layers=1, n_expert=8, top_k=2, expert_ff=128, shared_ff=128,
                    router_mode="sigmoid", router_bias=True, n_group=4, topk_group=2, route_scale=2.5),
        PRESETS["tiny-nemotron-h"](),          # Mamba-2 layers on the state-space scan kernel
        # glm5-next family: Kimi-delta-attention layers, hyper-connections around every sublayer, latent attention
        ModelConfig(arch="glm5_next", n_layer=3, hidden=256, vocab=1024, n_head=16, n_kv_head=16, head_dim=128,
                    layer_kinds=["kda", "kda", "mla"], kda_heads=4, kda_head_dim=64, kda_rank=32, hyper_streams=4,
                    hc_iters=8, q_lora=96, kv_lora=512, qk_nope_dim=64, qk_rope_dim=64, v_head_dim=64, qk_norm=False,
                    dense_ff=384, first_dense_layers=1, n_expert=8, top_k=2, expert_ff=128, shared_ff=128,
                    router_mode="sigmoid", router_bias=True, route_scale=2.0),
        PRESETS["tiny-qwen4exp"](),            # hybrid stack with gated hyper-connections in place of residual + pre-norms
        PRESETS["tiny-nemotron-h-moe"](),      # Mamba-2 + latent MoE with un-gated squared-ReLU experts
    ]


@pytest.mark.parametrize("idx", [0, 1, 2, 3, 4, 5, 6, 7])
@pytest.mark.parametrize("graphs", [False, True])
def test_gpu_engine_matches_cpu_logits(idx, graphs):
    """Greedy tokens of random tiny models are fragile under bf16; compare the first-step logits of the GPU
    forward against the CPU fp32 forward of the same (bf16-rounded) weights, then check the GPU engine runs."""
    cfg = _cfgs()[idx]
    w32 = {k: (v.bfloat16().float() if v.dtype == torch.float32 and v.dim() > 1 else v)
           for k, v in random_weights(cfg, "cpu", torch.float32, seed=3, std=0.05).items()}
    wgpu = {k: (v.bfloat16() if v.dim() > 1 and not k.endswith("conv_w") else v).cuda() for k, v in w32.items()}
    ec = dict(ctx_size=512, max_seqs=4, block_size=64, prefill_chunk=128, max_batch_tokens=256)
    cpu = build_engine(cfg, weights=w32, engine_cfg=EngineConfig(**ec), start=False)
    gpu = build_engine(cfg, weights=wgpu, device="cuda", engine_cfg=EngineConfig(cuda_graphs=graphs, **ec), start=False)
    prompt = torch.randint(0, 255, (150,), generator=torch.Generator().manual_seed(5)).tolist()
    outs = []
    for eng in (cpu, gpu):
        from legion_b200.engine.types import GenerateRequest, SamplingParams
        seq = eng.prepare(GenerateRequest(prompt_tokens=prompt, sampling=SamplingParams(max_tokens=4, ignore_eos=True)))
        eng.waiting.push(seq)
        eng._admit()
        b = eng.build_batch([(seq, 0, len(prompt))])
        outs.append(eng.model.forward(b, eng.kv, eng.states).logits.float().cpu())
    err = (outs[0] - outs[1]).abs().max().item()
    ref = outs[0].abs().max().item()
    assert err < 0.1 * ref + 0.1, (err, ref)
    gpu2 = build_engine(cfg, weights=wgpu, device="cuda", engine_cfg=EngineConfig(cuda_graphs=graphs, **ec))
    a = gpu2.generate_text(tokens=prompt, max_tokens=12, ignore_eos=True)
    b2 = gpu2.generate_text(tokens=prompt, max_tokens=12, ignore_eos=True)
    gpu2.shutdown()
    assert a.error is None and len(a.token_ids) == 12
    assert a.token_ids == b2.token_ids          # prefix-cache hit (and graph replay) reproduce the cold run
    assert b2.usage.cached_tokens >= 128
    from legion_b200.ops.sm100 import Workspace
    assert Workspace.get("cuda").check() == 0


def test_engine_with_nvfp4_experts():
    """Routed experts re-encoded to NVFP4 in HBM: first-step logits follow the run that uses the de-quantised copy
    of those weights expanded to bf16 (the two differ only in operand precision inside the expert GEMMs), and the
    engine generates through CUDA graphs with the 4-bit weights."""
    from legion_b200.config import ModelConfig
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    from legion_b200.models.weights import random_weights
    from legion_b200.ops.sm100 import Nv4Weight, QWeight, Workspace
    cfg = ModelConfig(arch="qwen3moe", n_layer=2, hidden=512, vocab=2048, n_head=8, n_kv_head=2, head_dim=128,
                      n_expert=8, top_k=2, expert_ff=256)
    w = random_weights(cfg, "cuda", torch.bfloat16, seed=0, std=0.05)
    ecfg = dict(ctx_size=512, max_seqs=2, block_size=64, prefill_chunk=256, prefix_cache=False)
    eng_q = build_engine(cfg, weights=dict(w), device="cuda", engine_cfg=EngineConfig(**ecfg), start=False)
    assert eng_q.model.quantize_experts_nvfp4() > 0
    w_deq = dict(w)
    for k, v in eng_q.model.w.items():
        if isinstance(v, (QWeight, Nv4Weight)):
            w_deq[k] = v.dequantize()
    eng_d = build_engine(cfg, weights=w_deq, device="cuda", engine_cfg=EngineConfig(**ecfg), start=False)
    prompt = list(range(3, 150))
    outs = []
    for eng in (eng_q, eng_d):
        seq = eng.prepare(GenerateRequest(prompt_tokens=prompt, sampling=SamplingParams(max_tokens=4, ignore_eos=True)))
        eng.waiting.push(seq)
        eng._admit()
        b = eng.build_batch([(seq, 0, len(prompt))])
        outs.append(eng.model.forward(b, eng.kv, eng.states).logits.float().cpu())
    err = (outs[0] - outs[1]).abs().max().item()
    ref = outs[1].abs().max().item()
    assert err < 0.03 * ref + 0.03, (err, ref)
    eng_g = build_engine(cfg, weights=dict(w), device="cuda", engine_cfg=EngineConfig(**ecfg))
    eng_g.model.quantize_experts_nvfp4()
    a = eng_g.generate_text(tokens=prompt, max_tokens=12, ignore_eos=True)
    b2 = eng_g.generate_text(tokens=prompt, max_tokens=12, ignore_eos=True)
    replays = eng_g._graphs.replays
    eng_g.shutdown()
    assert len(a.token_ids) == 12 and a.token_ids == b2.token_ids and replays > 0
    assert Workspace.get("cuda").check() == 0


def test_engine_with_fp8_weights():
    """All projection weights re-encoded to block-scaled FP8 (e4m3, 128 x 128 scales). Dense model: first-step
    logits stay close to the bf16 model's (weights and activations both lose precision; a routed model would also
    flip expert choices, so closeness is checked without routing). MoE model: the engine generates through CUDA
    graphs on the FP8 tensor-core path, reproducibly."""
    from legion_b200.config import ModelConfig
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    from legion_b200.models.weights import random_weights
    from legion_b200.ops.sm100 import Fp8Weight, Workspace
    ecfg = dict(ctx_size=512, max_seqs=2, block_size=64, prefill_chunk=256, prefix_cache=False)
    prompt = list(range(3, 150))
    dense = ModelConfig(arch="qwen3", n_layer=2, hidden=512, vocab=2048, n_head=8, n_kv_head=2, head_dim=128,
                        dense_ff=1024)
    w = random_weights(dense, "cuda", torch.bfloat16, seed=0, std=0.05)
    eng_q = build_engine(dense, weights=dict(w), device="cuda", engine_cfg=EngineConfig(**ecfg), start=False)
    assert eng_q.model.quantize_weights_fp8() > 0
    assert sum(isinstance(v, Fp8Weight) for v in eng_q.model.w.values()) == 4 * dense.n_layer
    eng_d = build_engine(dense, weights=dict(w), device="cuda", engine_cfg=EngineConfig(**ecfg), start=False)
    outs = []
    for eng in (eng_q, eng_d):
        seq = eng.prepare(GenerateRequest(prompt_tokens=prompt, sampling=SamplingParams(max_tokens=4, ignore_eos=True)))
        eng.waiting.push(seq)
        eng._admit()
        b = eng.build_batch([(seq, 0, len(prompt))])
        outs.append(eng.model.forward(b, eng.kv, eng.states).logits.float().cpu())
    err = (outs[0] - outs[1]).abs().max().item()
    ref = outs[1].abs().max().item()
    assert err < 0.15 * ref + 0.1, (err, ref)
    moe = ModelConfig(arch="qwen3moe", n_layer=2, hidden=512, vocab=2048, n_head=8, n_kv_head=2, head_dim=128,
                      n_expert=8, top_k=2, expert_ff=256)
    eng_g = build_engine(moe, weights=random_weights(moe, "cuda", torch.bfloat16, seed=0, std=0.05), device="cuda",
                         engine_cfg=EngineConfig(**ecfg))
    eng_g.model.quantize_weights_fp8()
    a = eng_g.generate_text(tokens=prompt, max_tokens=12, ignore_eos=True)
    b2 = eng_g.generate_text(tokens=prompt, max_tokens=12, ignore_eos=True)
    replays = eng_g._graphs.replays
    eng_g.shutdown()
    assert len(a.token_ids) == 12 and a.token_ids == b2.token_ids and replays > 0
    assert Workspace.get("cuda").check() == 0


def test_latent_attention_stacked_input_projection_and_shared_fp8_rows():
    """The query and latent projections of a latent-attention layer stacked into one GEMM give the logits of the
    separate GEMMs; with FP8 FFNs the shared and the routed experts read one encoding of the layer input, and the
    engine decodes through graphs on that path."""
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    from legion_b200.ops.sm100 import Fp8Weight, Workspace
    cfg = _cfgs()[3]
    w = random_weights(cfg, "cuda", torch.bfloat16, seed=3, std=0.05)
    ec = dict(ctx_size=512, max_seqs=4, block_size=64, prefill_chunk=256, prefix_cache=False)
    prompt = torch.randint(0, 255, (150,), generator=torch.Generator().manual_seed(5)).tolist()

    def first_logits(eng, toks=prompt):
        seq = eng.prepare(GenerateRequest(prompt_tokens=toks, sampling=SamplingParams(max_tokens=4, ignore_eos=True)))
        eng.waiting.push(seq)
        eng._admit()
        b = eng.build_batch([(seq, 0, len(toks))])
        return eng.model.forward(b, eng.kv, eng.states).logits.float().cpu()

    plain = build_engine(cfg, weights=dict(w), device="cuda", engine_cfg=EngineConfig(**ec), start=False)
    fused = build_engine(cfg, weights=dict(w), device="cuda", engine_cfg=EngineConfig(**ec), start=False)
    assert fused.model.fuse_mla_in_proj() == cfg.n_layer
    a, b = first_logits(plain), first_logits(fused)
    assert (a - b).abs().max().item() <= 0.02 * a.abs().max().item() + 1e-3
    # the key up-projection folded into the query projection (steps of at most 64 rows): same logits up to rounding
    assert fused.model.absorb_mla_q() == cfg.n_layer
    a, b = first_logits(plain, prompt[:40]), first_logits(fused, prompt[:40])
    assert (a - b).abs().max().item() <= 0.03 * a.abs().max().item() + 1e-3
    eng = build_engine(cfg, weights=dict(w), device="cuda", engine_cfg=EngineConfig(**ec))
    eng.model.fuse_mla_in_proj()
    eng.model.absorb_mla_q()
    assert eng.model.quantize_weights_fp8(ffn_only=True) > 0
    assert isinstance(eng.model.w["l1.moe.sh_gate_up"], Fp8Weight) and isinstance(eng.model.w["l1.mla.q_b"], torch.Tensor)
    r1 = eng.generate_text(tokens=prompt, max_tokens=12, ignore_eos=True)
    r2 = eng.generate_text(tokens=prompt, max_tokens=12, ignore_eos=True)
    replays = eng._graphs.replays
    eng.shutdown()
    assert len(r1.token_ids) == 12 and r1.token_ids == r2.token_ids and replays > 0
    assert Workspace.get("cuda").check() == 0


def test_prefix_cache_host_tier_on_gpu():
    """Evicted prefix-cache blocks go to pinned host memory and come back for a later prompt with that prefix."""
    from legion_b200.config import ModelConfig
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.models.weights import random_weights
    cfg = ModelConfig(arch="qwen3", n_layer=2, hidden=256, vocab=1024, n_head=4, n_kv_head=2, head_dim=128, dense_ff=512)
    w = random_weights(cfg, "cuda", torch.bfloat16, seed=0, std=0.05)
    ec = dict(ctx_size=512, max_seqs=1, block_size=64, prefill_chunk=256, kv_cache_tokens=640, prefix_cache=True)
    eng = build_engine(cfg, weights=dict(w), device="cuda", engine_cfg=EngineConfig(prefix_host_gib=0.05, **ec))
    pa = torch.randint(0, 255, (400,), generator=torch.Generator().manual_seed(1)).tolist()
    first = eng.generate_text(tokens=pa, max_tokens=6, ignore_eos=True)
    for sd in (2, 3):
        eng.generate_text(tokens=torch.randint(0, 255, (400,), generator=torch.Generator().manual_seed(sd)).tolist(),
                          max_tokens=6, ignore_eos=True)
    assert eng.stats().prefix_host_spilled > 0
    again = eng.generate_text(tokens=pa, max_tokens=6, ignore_eos=True)
    st = eng.stats()
    eng.shutdown()
    assert again.token_ids == first.token_ids
    assert st.prefix_host_restored > 0 and again.usage.cached_tokens >= 128


@pytest.mark.parametrize("quant", ["nvfp4", "nvfp4_ct", "fp8_block"])
def test_quantised_checkpoint_stays_in_its_shipped_encoding(tmp_path, quant):
    """An NVFP4 (ModelOpt or compressed-tensors) / block-FP8 directory loads with its expert and output projections
    still encoded: the code bytes are the file's, and the model's logits agree with the load that decodes to bf16."""
    from legion_b200.loaders.hf_map import load_hf, save_hf
    from legion_b200.loaders.safetensors_io import Checkpoint
    from legion_b200.ops import sm100
    cfg = ModelConfig(arch="qwen3moe", n_layer=2, hidden=256, vocab=1024, n_head=4, n_kv_head=2, head_dim=64,
                      n_expert=8, top_k=2, expert_ff=128)
    w = random_weights(cfg, "cpu", torch.float32, seed=2, std=0.05)
    d = str(tmp_path / "ck")
    save_hf(d, cfg, w, quant=quant)
    cfg_q, wq, ck = load_hf(d, "cuda", torch.bfloat16, keep_quant=True)
    cfg_d, wd, _ = load_hf(d, "cuda", torch.bfloat16)
    kind = sm100.Fp8Weight if quant == "fp8_block" else sm100.Nv4Weight
    for name in ("l0.moe.gate_up", "l1.moe.down", "l0.attn.o"):
        assert isinstance(wq[name], kind), (name, type(wq[name]))
        assert isinstance(wd[name], torch.Tensor)
    raw_name = "model.layers.0.mlp.experts.3.gate_proj.weight" + ("_packed" if quant == "nvfp4_ct" else "")
    raw = ck.get(raw_name).view(torch.uint8).cuda()
    got = wq["l0.moe.gate_up"].codes if quant != "fp8_block" else wq["l0.moe.gate_up"].data
    assert torch.equal(got[3, :raw.shape[0]], raw)
    # the de-quantised form of the kept encoding is the decoding load's tensor
    deq = wq["l0.moe.gate_up"].dequantize(torch.bfloat16).float()
    assert float((deq - wd["l0.moe.gate_up"].float()).abs().max()) <= 1e-2 * float(wd["l0.moe.gate_up"].float().abs().max())
    # and the model runs on it
    ec = dict(ctx_size=512, max_seqs=4, block_size=64, prefill_chunk=128, max_batch_tokens=256)
    prompt = torch.randint(0, 255, (90,), generator=torch.Generator().manual_seed(5)).tolist()
    outs = []
    for ww in (wd, wq):
        eng = build_engine(cfg_q, weights=ww, device="cuda", engine_cfg=EngineConfig(cuda_graphs=False, **ec), start=False)
        from legion_b200.engine.types import GenerateRequest, SamplingParams
        seq = eng.prepare(GenerateRequest(prompt_tokens=prompt, sampling=SamplingParams(max_tokens=4, ignore_eos=True)))
        eng.waiting.push(seq)
        eng._admit()
        b = eng.build_batch([(seq, 0, len(prompt))])
        outs.append(eng.model.forward(b, eng.kv, eng.states).logits.float().cpu())
    err = (outs[0] - outs[1]).abs().max().item()
    ref = outs[0].abs().max().item()
    assert err < (0.25 if quant != "fp8_block" else 0.1) * ref + 0.1, (err, ref)      # activations are quantised too
    assert sm100.Workspace.get("cuda").check() == 0


@pytest.mark.parametrize("idx", [0, 1, 2, 3, 4])
def test_decode_step_logits_from_the_cuda_graph_match_cpu(idx):
    """Steps 2+ of a generation replay a CUDA graph (packed input upload, decode kernels, LM head, arg-max). The
    logits the graph left behind for the LAST step are compared with the fp32 CPU model run over the same token
    history as one prompt: decode kernels, KV / recurrent state carried across steps and the graph's input
    packing all have to be right for them to agree."""
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    cfg = _cfgs()[idx]
    w32 = {k: (v.bfloat16().float() if v.dtype == torch.float32 and v.dim() > 1 else v)
           for k, v in random_weights(cfg, "cpu", torch.float32, seed=3, std=0.05).items()}
    wgpu = {k: (v.bfloat16() if v.dim() > 1 and not k.endswith("conv_w") else v).cuda() for k, v in w32.items()}
    ec = dict(ctx_size=512, max_seqs=4, block_size=64, prefill_chunk=128, max_batch_tokens=256, prefix_cache=False)
    gpu = build_engine(cfg, weights=wgpu, device="cuda", engine_cfg=EngineConfig(cuda_graphs=True, **ec), start=False)
    prompt = torch.randint(0, 255, (150,), generator=torch.Generator().manual_seed(7)).tolist()
    gpu.generate(GenerateRequest(prompt_tokens=prompt, sampling=SamplingParams(max_tokens=16, ignore_eos=True)))
    gpu._drain(block=False)
    for _ in range(40):
        gpu._admit()
        if gpu.running and len(gpu.running[0].tokens) >= len(prompt) + 5:
            break
        gpu.step()
    seq = gpu.running[0]
    assert gpu._graphs is not None and gpu._graphs.replays >= 3
    entry = next(iter(gpu._graphs.entries.values()))
    got = entry.logits[:1].float().cpu()
    history = list(seq.tokens[:-1])                    # the last step's input: everything before the token it picked
    assert int(got.argmax()) == seq.tokens[-1]
    cpu = build_engine(cfg, weights=w32, engine_cfg=EngineConfig(**ec), start=False)
    s2 = cpu.prepare(GenerateRequest(prompt_tokens=history, sampling=SamplingParams(max_tokens=2, ignore_eos=True)))
    cpu.waiting.push(s2)
    cpu._admit()
    rows, p0 = [], 0
    want = None
    while p0 < len(history):                           # chunked like any prompt; the last chunk's last row is the one
        n = min(128, len(history) - p0)
        out = cpu.model.forward(cpu.build_batch([(s2, p0, n)]), cpu.kv, cpu.states)
        want = out.logits[-1:].float()
        p0 += n
    err = (got - want).abs().max().item()
    ref = want.abs().max().item()
    assert err < 0.1 * ref + 0.1, (err, ref)
    from legion_b200.ops.sm100 import Workspace
    assert Workspace.get("cuda").check() == 0


@pytest.mark.parametrize("idx", [0, 1])
def test_speculative_verify_accepts_on_the_device(idx):
    """n-gram drafting on a GPU engine: verify steps take their (accepted drafts, next token) per sequence from the
    device-side accept kernel. The drafts of a repetitive prompt are accepted, and the greedy text equals the text
    of the same engine without drafting for as long as both pick the same token from (numerically slightly
    different) verify and decode kernels: the first divergence, if any, must come late."""
    cfg = _cfgs()[idx]
    w32 = random_weights(cfg, "cpu", torch.float32, seed=3, std=0.05)
    wgpu = {k: (v.bfloat16() if v.dim() > 1 and not k.endswith("conv_w") else v).cuda() for k, v in w32.items()}
    ec = dict(ctx_size=512, max_seqs=4, block_size=64, prefill_chunk=128, max_batch_tokens=256, prefix_cache=False)
    prompt = ([11, 12, 13, 14, 15, 16, 17, 18] * 12)[:90]
    plain = build_engine(cfg, weights=wgpu, device="cuda", engine_cfg=EngineConfig(**ec))
    a = plain.generate_text(tokens=prompt, max_tokens=24, ignore_eos=True)
    plain.shutdown()
    spec = build_engine(cfg, weights=wgpu, device="cuda", engine_cfg=EngineConfig(spec="ngram", spec_k=3, **ec))
    b = spec.generate_text(tokens=prompt, max_tokens=24, ignore_eos=True)
    st = spec.stats()
    spec.shutdown()
    assert a.error is None and b.error is None and len(b.token_ids) == 24
    if idx == 0:          # (the hybrid model's random text may offer the n-gram drafter nothing to propose)
        assert st.spec_verify_steps > 0 and st.spec_draft_tokens > 0
    same = 0
    for x, y in zip(a.token_ids, b.token_ids):
        if x != y:
            break
        same += 1
    assert same >= 8, (a.token_ids, b.token_ids)
    from legion_b200.ops.sm100 import Workspace
    assert Workspace.get("cuda").check() == 0


@pytest.mark.parametrize("idx", [0, 1])
def test_decode_step_as_two_concurrent_lanes_gives_the_same_tokens(idx):
    """From 64 rows a decode step's graph runs the two halves of the batch on parallel branches, each with its own
    workspace. Fifty greedy sequences must produce exactly the tokens of the single-lane graph."""
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    from legion_b200.ops import sm100
    cfg = _cfgs()[idx]
    w32 = random_weights(cfg, "cpu", torch.float32, seed=3, std=0.05)
    wgpu = {k: (v.bfloat16() if v.dim() > 1 and not k.endswith("conv_w") else v).cuda() for k, v in w32.items()}
    ec = dict(ctx_size=256, max_seqs=64, block_size=64, prefill_chunk=256, max_batch_tokens=2048, prefix_cache=False)
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, 255, (int(n),), generator=g).tolist() for n in torch.randint(5, 40, (50,), generator=g)]
    runs = []
    for lanes in (1, 2):
        old = sm100.TUNE["decode_lanes"]
        sm100.TUNE["decode_lanes"] = lanes
        try:
            eng = build_engine(cfg, weights=wgpu, device="cuda", engine_cfg=EngineConfig(**ec), start=False)
            streams = [eng.generate(GenerateRequest(prompt_tokens=p, sampling=SamplingParams(max_tokens=8, ignore_eos=True)))
                       for p in prompts]
            eng._drain(block=False)
            for _ in range(200):
                eng._admit()
                if not eng.running and len(eng.waiting) == 0:
                    break
                eng.step()
            runs.append([s.collect().token_ids for s in streams])
            assert eng._graphs.replays > 0
            assert (eng._graphs._lanes(64) == 2) == (lanes == 2)
            eng.shutdown()
        finally:
            sm100.TUNE["decode_lanes"] = old
    assert all(len(t) == 8 for t in runs[1])
    assert runs[0] == runs[1]
    assert sm100.Workspace.get("cuda").check() == 0


def test_memory_plan_auto_sizes_the_kv_pool_on_the_device():
    cfg = _cfgs()[1]
    w32 = random_weights(cfg, "cpu", torch.float32, seed=3, std=0.05)
    wgpu = {k: (v.bfloat16() if v.dim() > 1 and not k.endswith("conv_w") else v).cuda() for k, v in w32.items()}
    eng = build_engine(cfg, weights=wgpu, device="cuda", start=False,
                       engine_cfg=EngineConfig(ctx_size=512, max_seqs=4, block_size=64, kv_cache_tokens=-1))
    plan = eng.memory_plan
    assert plan is not None and plan.fits and plan.n_blocks == 4 * 512 // 64 == eng.pool.n_blocks
    assert plan.bytes_per_block == eng.kv.bytes_per_block() and plan.state_bytes > 0
    assert any("KV pool" in line for line in plan.lines())
    out = eng.generate_text(tokens=list(range(40)), max_tokens=4, ignore_eos=True) if eng.start() is None else None
    eng.shutdown()
    assert out.error is None and len(out.token_ids) == 4


def test_offloaded_experts_become_resident_on_the_device_and_decode_from_graphs():
    """Experts in pinned host memory behind a few HBM slots: the device-side cache step (victims by decayed heat,
    misses copied straight from mapped host memory, routing rewritten in slot numbers) first on its own against
    the host policy, then in the engine, where decode steps of the offloaded model replay CUDA graphs and produce
    the tokens of the all-resident model."""
    from legion_b200.ops import sm100
    from legion_b200.residency.experts import ExpertCache
    E, F, H = 24, 64, 128
    gu = (torch.arange(E, dtype=torch.float32)[:, None, None] + torch.rand(E, 2 * F, H)).bfloat16()
    dn = (torch.arange(E, dtype=torch.float32)[:, None, None] + torch.rand(E, H, F)).bfloat16()
    c = ExpertCache(gu, dn, n_slots=10, device="cuda")
    assert c.graph_safe
    g = torch.Generator().manual_seed(0)
    for step in range(12):
        ids = torch.stack([torch.randperm(E, generator=g)[:2] for _ in range(4)]).int().cuda()
        slots = c.prepare(ids)
        assert sm100.Workspace.get("cuda").check() == 0
        sg, sd = c.weights()
        for t in range(4):
            for j in range(2):
                e, s = int(ids[t, j]), int(slots[t, j])
                assert torch.equal(sg[s].cpu(), gu[e]) and torch.equal(sd[s].cpu(), dn[e]), (step, e, s)
    st = c.sync_stats()
    assert st.misses > 0 and st.hits > 0 and st.steps == 12 and st.bytes_copied == st.misses * c.bytes_per_expert
    assert sorted(x for x in c.expert_in if x >= 0) == sorted(e for e in range(E) if c.slot_of[e] >= 0)
    # more experts in one step than slots: reported through the status word, no hang
    c.prepare(torch.arange(12, dtype=torch.int32).view(1, 12).cuda())
    assert sm100.Workspace.get("cuda").check() != 0
    # engine: offloaded == resident, decode from graphs (prompt chunks of 4 tokens route to at most 8 of 32 experts)
    cfg = ModelConfig(arch="qwen3moe", n_layer=2, hidden=256, vocab=1024, n_head=4, n_kv_head=2, head_dim=64,
                      n_expert=32, top_k=2, expert_ff=128)
    w32 = random_weights(cfg, "cpu", torch.float32, seed=3, std=0.05)
    wgpu = {k: (v.bfloat16() if v.dim() > 1 else v).cuda() for k, v in w32.items()}
    ec = dict(ctx_size=256, max_seqs=2, block_size=64, prefill_chunk=4, max_batch_tokens=4, prefix_cache=False)
    prompt = torch.randint(0, 255, (30,), generator=torch.Generator().manual_seed(1)).tolist()
    a = build_engine(cfg, weights=dict(wgpu), device="cuda", engine_cfg=EngineConfig(**ec))
    want = a.generate_text(tokens=prompt, max_tokens=10, ignore_eos=True).token_ids
    a.shutdown()
    b = build_engine(cfg, weights=dict(wgpu), device="cuda", engine_cfg=EngineConfig(**ec), start=False)
    b.model.offload_experts(n_slots=12)
    assert b._graphs is not None and all(cache.graph_safe for cache in b.model.expert_cache.values())
    b.start()
    got = b.generate_text(tokens=prompt, max_tokens=10, ignore_eos=True).token_ids
    replays = b._graphs.replays
    misses = sum(cache.sync_stats().misses for cache in b.model.expert_cache.values())
    b.shutdown()
    assert got == want and replays > 0 and misses > 0
    assert sm100.Workspace.get("cuda").check() == 0


def test_images_on_gpu_match_the_cpu_engine_and_decode_from_graphs():
    """A prompt with an image on the GPU engine (tower in bf16 on the device, image rows spliced into the token
    embedding, per-token rotary rows for the three position axes, extra rows after the first layer): first-step
    logits close to the fp32 CPU engine's, and graph-replayed decode steps take the shifted rotary positions."""
    import io
    from PIL import Image
    from legion_b200.engine.types import ChatMessage, GenerateRequest, SamplingParams
    from legion_b200.vision import VisionConfig, VisionHparams, VisionRuntime, VisionTower, random_vision_weights
    im = Image.new("RGB", (64, 48), (180, 40, 90))
    for x in range(0, 64, 5):
        im.putpixel((x, (x * 3) % 48), (x * 4 % 256, 200, 10))
    buf = io.BytesIO()
    im.save(buf, "PNG")
    img = buf.getvalue()
    cfg = ModelConfig(arch="qwen3", n_layer=3, hidden=256, vocab=1024, n_head=4, n_kv_head=2, head_dim=64, dense_ff=512,
                      mrope_sections=(11, 11, 10))
    w32 = {k: (v.bfloat16().float() if v.dim() > 1 else v)
           for k, v in random_weights(cfg, "cpu", torch.float32, seed=3, std=0.05).items()}
    wgpu = {k: (v.bfloat16() if v.dim() > 1 else v).cuda() for k, v in w32.items()}
    vc = VisionConfig(depth=2, hidden=64, n_head=2, intermediate=96, out_hidden=256, patch_size=8, num_pos=16,
                      deepstack_layers=(0,))
    vw = {k: v.bfloat16().float() for k, v in random_vision_weights(vc, seed=5).items()}
    hp = dict(patch_size=8, spatial_merge_size=2, min_tokens=2, max_tokens=64)
    ec = dict(ctx_size=512, max_seqs=4, block_size=64, prefill_chunk=256)
    msg = ChatMessage("user", [{"type": "image"}, {"type": "text", "text": "describe"}])
    outs = []
    engs = []
    for dev, ww, vww in (("cpu", w32, vw), ("cuda", wgpu, {k: v.bfloat16().cuda() for k, v in vw.items()})):
        eng = build_engine(cfg, weights=dict(ww), device=dev, engine_cfg=EngineConfig(**ec), start=False)
        eng.attach_vision(VisionRuntime(VisionTower(vc, vww), VisionHparams(**hp)))
        seq = eng.prepare(GenerateRequest(messages=[msg], images=[img], sampling=SamplingParams(max_tokens=4)))
        eng.waiting.push(seq)
        eng._admit()
        b = eng.build_batch([(seq, 0, len(seq.tokens))])
        assert b.embeds is not None and b.rope_table is not None and b.deepstack is not None
        outs.append(eng.model.forward(b, eng.kv, eng.states).logits.float().cpu())
        engs.append(eng)
    err = (outs[0] - outs[1]).abs().max().item()
    assert err < 0.1 * outs[0].abs().max().item() + 0.1, err
    gpu = build_engine(cfg, weights=dict(wgpu), device="cuda", engine_cfg=EngineConfig(**ec))
    gpu.attach_vision(VisionRuntime(VisionTower(vc, {k: v.bfloat16().cuda() for k, v in vw.items()}), VisionHparams(**hp)))
    req = lambda: GenerateRequest(messages=[msg], images=[img], sampling=SamplingParams(max_tokens=10, ignore_eos=True))
    r1 = gpu.generate(req()).collect()
    r2 = gpu.generate(req()).collect()
    plain = build_engine(cfg, weights=dict(wgpu), device="cuda", engine_cfg=EngineConfig(cuda_graphs=False, **ec))
    plain.attach_vision(VisionRuntime(VisionTower(vc, {k: v.bfloat16().cuda() for k, v in vw.items()}), VisionHparams(**hp)))
    r3 = plain.generate(req()).collect()
    replays = gpu._graphs.replays
    gpu.shutdown()
    plain.shutdown()
    assert r1.error is None and r1.token_ids == r2.token_ids == r3.token_ids and replays > 0
