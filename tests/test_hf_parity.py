"""The model code against an independent implementation: tiny random checkpoints built and saved by the
``transformers`` package's own modelling code are read through the HF loader, and the prompt's logits at every
position plus a greedy continuation (decoded through the engine with chunked prefill and the paged cache) must match
what ``transformers`` computes. Families: llama, qwen3_moe, deepseek_v3 (latent attention, grouped sigmoid router with
bias), qwen3_next (fused, interleaved DeltaNet projections), qwen3_5 and qwen3_5_moe (Gated DeltaNet hybrid; the
flagship family)."""
import pytest
import torch

from legion_b200.engine.lm import EngineConfig, build_engine
from legion_b200.engine.types import GenerateRequest, SamplingParams
from legion_b200.loaders.hf_map import load_hf

transformers = pytest.importorskip("transformers")

HYBRID = dict(vocab_size=320, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, linear_conv_kernel_dim=4, linear_key_head_dim=8, linear_value_head_dim=8,
              linear_num_key_heads=2, linear_num_value_heads=4, max_position_embeddings=256, full_attention_interval=4)
FAMILIES = {
    "llama": ("llama", "LlamaConfig", "LlamaForCausalLM",
              dict(vocab_size=320, hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                   intermediate_size=96, max_position_embeddings=256)),
    "qwen3": ("qwen3", "Qwen3Config", "Qwen3ForCausalLM",
              dict(vocab_size=320, hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                   head_dim=24, intermediate_size=96, max_position_embeddings=256, tie_word_embeddings=True)),
    "qwen3_moe": ("qwen3_moe", "Qwen3MoeConfig", "Qwen3MoeForCausalLM",
                  dict(vocab_size=320, hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                       head_dim=16, moe_intermediate_size=32, num_experts_per_tok=2, num_experts=8, norm_topk_prob=True,
                       max_position_embeddings=256, intermediate_size=96, decoder_sparse_step=1, mlp_only_layers=[])),
    # a leading dense layer, router weights left un-normalised
    "qwen3_moe_dense_first": ("qwen3_moe", "Qwen3MoeConfig", "Qwen3MoeForCausalLM",
                              dict(vocab_size=320, hidden_size=64, num_hidden_layers=3, num_attention_heads=4,
                                   num_key_value_heads=2, head_dim=16, moe_intermediate_size=32, num_experts_per_tok=2,
                                   num_experts=8, norm_topk_prob=False, max_position_embeddings=256,
                                   intermediate_size=96, decoder_sparse_step=1, mlp_only_layers=[0])),
    "deepseek_v3": ("deepseek_v3", "DeepseekV3Config", "DeepseekV3ForCausalLM",
                    dict(vocab_size=320, hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4,
                         intermediate_size=96, moe_intermediate_size=32, n_shared_experts=1, n_routed_experts=8,
                         routed_scaling_factor=2.5, kv_lora_rank=16, q_lora_rank=24, qk_rope_head_dim=8, v_head_dim=16,
                         qk_nope_head_dim=16, n_group=2, topk_group=1, num_experts_per_tok=2, first_k_dense_replace=1,
                         norm_topk_prob=True, max_position_embeddings=256)),
    # rotary scaling as real checkpoints use it: Llama-3.1's frequency-dependent scaling, DeepSeek's YaRN (which also
    # scales the softmax by the square of its all-dimension term)
    "llama_scaled": ("llama", "LlamaConfig", "LlamaForCausalLM",
                     dict(vocab_size=320, hidden_size=64, num_hidden_layers=3, num_attention_heads=4,
                          num_key_value_heads=2, intermediate_size=96, max_position_embeddings=256,
                          rope_parameters={"rope_type": "llama3", "rope_theta": 10000.0, "factor": 8.0,
                                           "original_max_position_embeddings": 32, "low_freq_factor": 1.0,
                                           "high_freq_factor": 4.0})),
    "deepseek_v3_yarn": ("deepseek_v3", "DeepseekV3Config", "DeepseekV3ForCausalLM",
                         dict(vocab_size=320, hidden_size=64, num_hidden_layers=3, num_attention_heads=4,
                              num_key_value_heads=4, intermediate_size=96, moe_intermediate_size=32, n_shared_experts=1,
                              n_routed_experts=8, routed_scaling_factor=2.5, kv_lora_rank=16, q_lora_rank=24,
                              qk_rope_head_dim=8, v_head_dim=16, qk_nope_head_dim=16, n_group=2, topk_group=1,
                              num_experts_per_tok=2, first_k_dense_replace=1, norm_topk_prob=True,
                              max_position_embeddings=256,
                              rope_parameters={"rope_type": "yarn", "rope_theta": 10000.0, "factor": 8.0,
                                               "original_max_position_embeddings": 32, "beta_fast": 32, "beta_slow": 1,
                                               "mscale": 1.0, "mscale_all_dim": 1.0})),
    "qwen3_next": ("qwen3_next", "Qwen3NextConfig", "Qwen3NextForCausalLM",
                   dict(HYBRID, moe_intermediate_size=32, shared_expert_intermediate_size=32, num_experts_per_tok=2,
                        num_experts=8, intermediate_size=96, decoder_sparse_step=1, mlp_only_layers=[],
                        norm_topk_prob=True)),
    "qwen3_5": ("qwen3_5", "Qwen3_5TextConfig", "Qwen3_5ForCausalLM", dict(HYBRID, intermediate_size=96)),
    "qwen3_5_moe": ("qwen3_5_moe", "Qwen3_5MoeTextConfig", "Qwen3_5MoeForCausalLM",
                    dict(HYBRID, moe_intermediate_size=32, shared_expert_intermediate_size=32, num_experts_per_tok=2,
                         num_experts=8)),
}


def _tiny_checkpoint(name, path):
    import importlib
    mod, cfg_cls, model_cls, kw = FAMILIES[name]
    try:
        pkg = importlib.import_module(f"transformers.models.{mod}")
        modelling = importlib.import_module(f"transformers.models.{mod}.modeling_{mod}")
    except ImportError:
        pytest.skip(f"this transformers has no {mod}")
    hc = getattr(pkg, cfg_cls)(**kw, pad_token_id=0, eos_token_id=1, bos_token_id=2)
    hc._attn_implementation = "eager"
    torch.manual_seed(0)
    m = getattr(modelling, model_cls)(hc).eval().float()
    zero_centred = name.startswith(("qwen3_5", "qwen3_next"))          # this family stores norm weights as (w - 1)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" in n and p.dim() == 1:
                base = 0.0 if zero_centred and "linear_attn.norm" not in n else 1.0
                p.copy_(base + 0.2 * torch.randn_like(p))
            elif n.endswith("A_log"):
                p.copy_(torch.randn_like(p) * 0.5)
            elif n.endswith("dt_bias"):
                p.copy_(torch.randn_like(p) * 0.3)
            elif p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.08)
        for n, b in m.named_buffers():
            if n.endswith("e_score_correction_bias"):
                b.copy_(torch.randn_like(b) * 0.3)
    m.save_pretrained(str(path), safe_serialization=True)
    return m


@pytest.mark.parametrize("name", list(FAMILIES))
def test_logits_and_greedy_tokens_match_transformers(tmp_path, name):
    m = _tiny_checkpoint(name, tmp_path)
    n = 40
    ids = torch.randint(3, 320, (1, n), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        ref = m(input_ids=ids).logits[0].float()
        cont = m.generate(ids, max_new_tokens=6, do_sample=False)[0, n:].tolist()
    cfg, w, _ = load_hf(str(tmp_path), "cpu", torch.float32)
    ec = dict(ctx_size=128, max_seqs=2, block_size=16, max_batch_tokens=128)
    eng = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(**ec), start=False)
    seq = eng.prepare(GenerateRequest(prompt_tokens=ids[0].tolist(), sampling=SamplingParams(max_tokens=1)))
    eng.waiting.push(seq)
    eng._admit()
    b = eng.build_batch([(seq, 0, n)])
    b.logit_rows = None
    with torch.no_grad():
        mine = eng.model.forward(b, eng.kv, eng.states).logits.float()
    assert (mine - ref).abs().max().item() < 2e-4
    eng2 = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(prefill_chunk=16, **ec))
    out = eng2.generate_text(tokens=ids[0].tolist(), max_tokens=6, ignore_eos=True).token_ids
    eng2.shutdown()
    assert out == cont


@pytest.mark.parametrize("latent", [False, True])
def test_nemotron_h_blocks_match_transformers(tmp_path, latent):
    """Nemotron-H as its checkpoints lay it out (one sub-layer per block: Mamba-2 with two norm groups, attention
    without rotary embedding, MoE with a grouped sigmoid router, selection bias, shared expert and optional latent
    projections) against ``transformers``' implementation. Its scan runs as one chunk here: across chunk boundaries
    that package's pure-PyTorch scan disagrees with its own single-chunk and step forms."""
    try:
        from transformers.models.nemotron_h import NemotronHConfig
        from transformers.models.nemotron_h.modeling_nemotron_h import NemotronHForCausalLM
    except ImportError:
        pytest.skip("this transformers has no nemotron_h")
    torch.manual_seed(0)
    hc = NemotronHConfig(vocab_size=320, hidden_size=64, layers_block_type=["mamba", "moe", "attention", "moe", "mamba", "moe"],
                         num_attention_heads=4, num_key_value_heads=2, head_dim=16, max_position_embeddings=256,
                         intermediate_size=96, ssm_state_size=16, mamba_num_heads=8, mamba_head_dim=8, n_groups=2,
                         conv_kernel=4, chunk_size=64, n_routed_experts=8, n_shared_experts=1, moe_intermediate_size=32,
                         moe_shared_expert_intermediate_size=48, moe_latent_size=24 if latent else None,
                         num_experts_per_tok=2, routed_scaling_factor=2.5, n_group=2, topk_group=1, norm_topk_prob=True,
                         use_mamba_kernels=False, pad_token_id=0, bos_token_id=1, eos_token_id=2)
    hc._attn_implementation = "eager"
    m = NemotronHForCausalLM(hc).eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith("A_log"):
                p.copy_(torch.randn_like(p) * 0.5)
            elif n.endswith("dt_bias") or n.endswith(".D") or n.endswith("conv1d.bias"):
                p.copy_(torch.randn_like(p) * 0.3)
            elif "norm" in n and p.dim() == 1:
                p.copy_(1.0 + 0.2 * torch.randn_like(p))
            elif p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.08)
        for n, b in m.named_buffers():
            if n.endswith("e_score_correction_bias"):
                b.copy_(torch.randn_like(b) * 0.3)
    m.save_pretrained(str(tmp_path), safe_serialization=True)
    n = 40
    ids = torch.randint(3, 320, (1, n), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        ref = m(input_ids=ids).logits[0].float()
        cont = m.generate(ids, max_new_tokens=6, do_sample=False)[0, n:].tolist()
    cfg, w, _ = load_hf(str(tmp_path), "cpu", torch.float32)
    assert cfg.block_form and cfg.layer_kinds == ["mamba2", "moe", "nope", "moe", "mamba2", "moe"]
    assert cfg.moe_latent == (24 if latent else 0) and cfg.ssm_groups == 2
    ec = dict(ctx_size=128, max_seqs=2, block_size=16, max_batch_tokens=128)
    eng = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(**ec), start=False)
    seq = eng.prepare(GenerateRequest(prompt_tokens=ids[0].tolist(), sampling=SamplingParams(max_tokens=1)))
    eng.waiting.push(seq)
    eng._admit()
    b = eng.build_batch([(seq, 0, n)])
    b.logit_rows = None
    with torch.no_grad():
        mine = eng.model.forward(b, eng.kv, eng.states).logits.float()
    assert (mine - ref).abs().max().item() < 2e-4
    eng2 = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(prefill_chunk=16, **ec))
    out = eng2.generate_text(tokens=ids[0].tolist(), max_tokens=6, ignore_eos=True).token_ids
    # the same model through batching and the prefix cache: engine invariants hold for the block form too
    again = eng2.generate_text(tokens=ids[0].tolist(), max_tokens=6, ignore_eos=True).token_ids
    eng2.shutdown()
    assert out == cont and again == cont


def test_qwen3_vl_moe_text_path_matches_transformers(tmp_path):
    """The language model of a Qwen3-VL-MoE checkpoint (weights under ``model.language_model.``, experts stored fused
    as ``experts.gate_up_proj`` [E, 2F, H], multi-section rotary configuration) on a text prompt; sized so that 2F
    equals the hidden width, where the fused tensor alone cannot tell its layout."""
    try:
        from transformers.models.qwen3_vl_moe.configuration_qwen3_vl_moe import Qwen3VLMoeConfig
        from transformers.models.qwen3_vl_moe.modeling_qwen3_vl_moe import Qwen3VLMoeForConditionalGeneration
    except ImportError:
        pytest.skip("this transformers has no qwen3_vl_moe")
    torch.manual_seed(0)
    conf = Qwen3VLMoeConfig(
        text_config=dict(vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=3, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=32, max_position_embeddings=512, moe_intermediate_size=32,
                         num_experts=8, num_experts_per_tok=2, decoder_sparse_step=1, mlp_only_layers=[],
                         norm_topk_prob=True, pad_token_id=0, eos_token_id=1, bos_token_id=2,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [6, 5, 5],
                                          "mrope_interleaved": True}),
        vision_config=dict(depth=2, hidden_size=32, num_heads=4, intermediate_size=48, out_hidden_size=64, patch_size=4,
                           temporal_patch_size=2, spatial_merge_size=2, num_position_embeddings=36,
                           deepstack_visual_indexes=[0], hidden_act="gelu_pytorch_tanh", in_channels=3),
        image_token_id=300, video_token_id=303, vision_start_token_id=301, vision_end_token_id=302,
        tie_word_embeddings=False)
    for c in (conf, conf.text_config, conf.vision_config):
        c._attn_implementation = "eager"
    m = Qwen3VLMoeForConditionalGeneration(conf).eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.08)
            elif "norm" in n and n.endswith("weight"):
                p.copy_(1.0 + 0.2 * torch.randn_like(p))
    m.save_pretrained(str(tmp_path), safe_serialization=True)
    ids = torch.randint(3, 299, (1, 30), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        ref = m(input_ids=ids).logits[0].float()
    cfg, w, _ = load_hf(str(tmp_path), "cpu", torch.float32)
    assert cfg.arch == "qwen3moe" and cfg.n_expert == 8 and cfg.mrope_sections == (6, 5, 5)
    eng = build_engine(cfg, weights=dict(w), start=False,
                       engine_cfg=EngineConfig(ctx_size=128, max_seqs=2, block_size=16, max_batch_tokens=128))
    seq = eng.prepare(GenerateRequest(prompt_tokens=ids[0].tolist(), sampling=SamplingParams(max_tokens=1)))
    eng.waiting.push(seq)
    eng._admit()
    b = eng.build_batch([(seq, 0, 30)])
    b.logit_rows = None
    with torch.no_grad():
        mine = eng.model.forward(b, eng.kv, eng.states).logits.float()
    assert (mine - ref).abs().max().item() < 2e-4
