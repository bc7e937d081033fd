"""GGUF <-> engine mapping: metadata keys to ``ModelConfig`` and GGUF tensor names to the canonical
fused weight names (and back, for writing GGUF files of our own models).

Schema per the reference's hybrid-MoE architecture (``src/model/qwen35/mod.rs:60-98``,
``src/hf/qwen35.rs:321-392``): ``{arch}.block_count``, ``.embedding_length``, ``.attention.head_count(_kv)``,
``.attention.key_length``, ``.rope.dimension_count``, ``.rope.freq_base``, ``.expert_count``,
``.expert_used_count``, ``.full_attention_interval``, ``.ssm.conv_kernel`` / ``.state_size`` (key head dim) /
``.group_count`` (key heads) / ``.time_step_rank`` (value heads) / ``.inner_size``; tensors ``blk.N.attn_q``
(q and gate interleaved per head for gated attention), ``attn_qkv`` + ``attn_gate`` (z) + ``ssm_alpha`` /
``ssm_beta`` + ``ssm_conv1d`` + ``ssm_dt.bias`` + ``ssm_a`` + ``ssm_norm`` + ``ssm_out`` for DeltaNet layers,
``ffn_gate_inp`` (router), ``ffn_{gate,up,down}_exps`` (stacked), ``ffn_*_shexp``, ``ffn_gate_inp_shexp``.
In GGUF files DeltaNet value heads are in tiled order (value head h reads key head h % n_k).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config import ModelConfig
from ..models.weights import is_fp32_weight, weight_shapes
from .gguf import GgufFile, GgufWriter

ARCH_TO_GGUF = {"qwen35moe": "qwen35moe", "qwen35": "qwen35", "qwen3moe": "qwen3moe", "qwen3": "qwen3",
                "llama": "llama", "deepseek_v3": "deepseek2", "gemma4": "gemma4", "nemotron_h": "nemotron_h"}
GGUF_TO_ARCH = {v: k for k, v in ARCH_TO_GGUF.items()}
GGUF_TO_ARCH["nemotron_h_moe"] = "nemotron_h"


def _gemma4_config(md: dict) -> ModelConfig:
    """Gemma 4 (``gemma4.*`` keys as the reference reads them, ``src/model/gemma4.rs::parse``): per-layer
    sliding-window pattern and kv-head counts, head sizes and rotary bases per layer kind, shared KV layers,
    per-layer embedding width, soft cap."""
    g = lambda k, d=None: md.get(f"gemma4.{k}", d)        # noqa: E731
    n_layer = int(g("block_count"))
    swa = [bool(v) for v in g("attention.sliding_window_pattern")][:n_layer]

    def per_layer(key):
        v = g(key)
        return [int(x) for x in v][:n_layer] if isinstance(v, (list, tuple)) else [int(v)] * n_layer

    kvh, ff = per_layer("attention.head_count_kv"), per_layer("feed_forward_length")
    kv_swa = {kvh[i] for i in range(n_layer) if swa[i]} or {1}
    kv_full = {kvh[i] for i in range(n_layer) if not swa[i]} or {1}
    if len(kv_swa) > 1 or len(kv_full) > 1:
        raise ValueError("gemma4: kv-head counts must be uniform per layer kind")
    hidden, head_dim = int(g("embedding_length")), int(g("attention.key_length"))
    n_expert = int(g("expert_count", 0))
    return ModelConfig(
        arch="gemma4", n_layer=n_layer, hidden=hidden, n_head=int(g("attention.head_count")), n_kv_head=kv_full.pop(),
        head_dim=head_dim, layer_kinds=["swa" if s_ else "attn" for s_ in swa],
        sliding_window=int(g("attention.sliding_window")), rope_dim=int(g("rope.dimension_count", head_dim)),
        rope_theta=float(g("rope.freq_base", 10000.0)), swa_head_dim=int(g("attention.key_length_swa")),
        swa_kv_heads=kv_swa.pop(), rope_theta_swa=float(g("rope.freq_base_swa", g("rope.freq_base", 10000.0))),
        rms_eps=float(g("attention.layer_norm_rms_epsilon", 1e-6)), max_position=int(g("context_length", 131072)),
        vocab=len(md.get("tokenizer.ggml.tokens", [])) or 0, ffn_act="gelu_tanh", dense_ff=max(ff), tie_embeddings=True,
        logit_softcap=float(g("final_logit_softcapping", 0.0)), attn_scale=1.0, sandwich_norm=True,
        embed_scale=float(hidden) ** 0.5, v_norm=True, kv_shared_layers=int(g("attention.shared_kv_layers", 0)),
        ple_dim=int(g("embedding_length_per_layer_input", 0)), n_expert=n_expert,
        top_k=int(g("expert_used_count", 0)), expert_ff=int(g("expert_feed_forward_length", 0)),
        router_mode="softmax", norm_topk=True)


def _nemotron_arch(cfg: ModelConfig) -> str:
    return "nemotron_h_moe" if "moe" in cfg.layer_kinds else "nemotron_h"


def _nemotron_config(md: dict, a: str) -> ModelConfig:
    """Nemotron-H (``nemotron_h`` / ``nemotron_h_moe`` keys as the reference reads them,
    ``src/model/nemotron_h.rs::parse``): one sub-layer per block, its kind told by the per-layer kv-head and FFN-size
    arrays (neither: Mamba-2; kv heads only: attention; an FFN size: FFN or MoE)."""
    g = lambda k, d=None: md.get(f"{a}.{k}", d)        # noqa: E731
    n_layer = int(g("block_count")) - int(g("nextn_predict_layers", 0))

    def per_layer(key):
        v = g(key, 0)
        return [int(x) for x in v][:n_layer] if isinstance(v, (list, tuple)) else [int(v)] * n_layer

    kvh, ff = per_layer("attention.head_count_kv"), per_layer("feed_forward_length")
    moe = a == "nemotron_h_moe"
    kinds = ["mamba2" if (k == 0 and f == 0) else "nope" if f == 0 else ("moe" if moe else "ffn") for k, f in zip(kvh, ff)]
    heads, inner = int(g("ssm.time_step_rank")), int(g("ssm.inner_size"))
    hidden, n_head = int(g("embedding_length")), int(g("attention.head_count"))
    kw = dict(arch="nemotron_h", n_layer=n_layer, hidden=hidden, n_head=n_head, n_kv_head=max(kvh) or n_head,
              head_dim=int(g("attention.key_length", hidden // n_head)), layer_kinds=kinds, block_form=True, qk_norm=False,
              ffn_act="relu2", rms_eps=float(g("attention.layer_norm_rms_epsilon", g("attention.layer_norm_epsilon", 1e-5))),
              max_position=int(g("context_length", 4096)), vocab=len(md.get("tokenizer.ggml.tokens", [])) or 0,
              ssm_state=int(g("ssm.state_size")), ssm_heads=heads, ssm_head_dim=inner // heads,
              ssm_groups=int(g("ssm.group_count", 1)), ssm_conv=int(g("ssm.conv_kernel", 4)))
    sizes = [f for f in ff if f]
    if moe:
        kw.update(n_expert=int(g("expert_count")), top_k=max(per_layer("expert_used_count")), expert_ff=sizes[0] if sizes else 0,
                  shared_ff=int(g("expert_shared_feed_forward_length", 0)), moe_latent=int(g("moe_latent_size", 0)),
                  router_mode="sigmoid", router_bias=True, norm_topk=bool(g("expert_weights_norm", False)),
                  route_scale=float(g("expert_weights_scale", 0.0)) or 1.0)
    else:
        kw["dense_ff"] = sizes[0] if sizes else 0
    return ModelConfig(**kw)


def _nemotron_metadata(cfg: ModelConfig) -> Dict[str, object]:
    a = _nemotron_arch(cfg)
    ff = cfg.expert_ff if a == "nemotron_h_moe" else cfg.dense_ff
    md = {f"{a}.block_count": cfg.n_layer, f"{a}.embedding_length": cfg.hidden, f"{a}.attention.head_count": cfg.n_head,
          f"{a}.attention.head_count_kv": [cfg.n_kv_head if k == "nope" else 0 for k in cfg.layer_kinds],
          f"{a}.feed_forward_length": [cfg.dense_ff if k == "ffn" else ff if k == "moe" else 0 for k in cfg.layer_kinds],
          f"{a}.attention.key_length": cfg.head_dim, f"{a}.attention.value_length": cfg.head_dim,
          f"{a}.attention.layer_norm_rms_epsilon": float(cfg.rms_eps), f"{a}.context_length": cfg.max_position,
          f"{a}.ssm.conv_kernel": cfg.ssm_conv, f"{a}.ssm.state_size": cfg.ssm_state, f"{a}.ssm.group_count": cfg.ssm_groups,
          f"{a}.ssm.time_step_rank": cfg.ssm_heads, f"{a}.ssm.inner_size": cfg.ssm_heads * cfg.ssm_head_dim,
          f"{a}.vocab_size": cfg.vocab}
    if a == "nemotron_h_moe":
        md.update({f"{a}.expert_count": cfg.n_expert, f"{a}.expert_used_count": cfg.top_k,
                   f"{a}.expert_shared_feed_forward_length": cfg.shared_ff, f"{a}.expert_weights_norm": bool(cfg.norm_topk),
                   f"{a}.expert_weights_scale": float(cfg.route_scale), f"{a}.expert_gating_func": 2})
        if cfg.moe_latent:
            md[f"{a}.moe_latent_size"] = cfg.moe_latent
    return md


_NEMOTRON_TENSORS = {
    "mamba2": (("ssm.in", "ssm_in.weight"), ("ssm.conv_w", "ssm_conv1d.weight"), ("ssm.conv_b", "ssm_conv1d.bias"),
               ("ssm.dt_bias", "ssm_dt.bias"), ("ssm.A", "ssm_a"), ("ssm.D", "ssm_d"), ("ssm.norm", "ssm_norm.weight"),
               ("ssm.out", "ssm_out.weight")),
    "nope": (("attn.o", "attn_output.weight"),),
    "ffn": (("mlp.gate_up", "ffn_up.weight"), ("mlp.down", "ffn_down.weight")),
    "moe": (("moe.router", "ffn_gate_inp.weight"), ("moe.router_bias", "exp_probs_b.bias"),
            ("moe.gate_up", "ffn_up_exps.weight"), ("moe.down", "ffn_down_exps.weight"),
            ("moe.sh_gate_up", "ffn_up_shexp.weight"), ("moe.sh_down", "ffn_down_shexp.weight"),
            ("moe.lat_down", "ffn_latent_down.weight"), ("moe.lat_up", "ffn_latent_up.weight")),
}


def _nemotron_to_gguf(cfg: ModelConfig, w: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {"token_embd.weight": w["tok_embd"], "output_norm.weight": w["output_norm"]}
    if "output" in w:
        out["output.weight"] = w["output"]
    nq, nk = cfg.n_head * cfg.head_dim, cfg.n_kv_head * cfg.head_dim
    for il, kind in enumerate(cfg.layer_kinds):
        p, b = f"l{il}", f"blk.{il}"
        out[f"{b}.attn_norm.weight"] = w[f"{p}.attn_norm"]
        for ours, theirs in _NEMOTRON_TENSORS[kind]:
            if f"{p}.{ours}" in w:
                t = w[f"{p}.{ours}"]
                if ours in ("ssm.A", "ssm.D"):
                    t = t.reshape(1, -1)
                elif ours == "ssm.norm":
                    t = t.reshape(cfg.ssm_groups, -1)
                out[f"{b}.{theirs}"] = t
        if kind == "nope":
            qkv = w[f"{p}.attn.qkv"]
            out[f"{b}.attn_q.weight"], out[f"{b}.attn_k.weight"] = qkv[:nq], qkv[nq:nq + nk]
            out[f"{b}.attn_v.weight"] = qkv[nq + nk:]
    return out


def _nemotron_from_gguf(cfg: ModelConfig, get, has) -> Dict[str, torch.Tensor]:
    w: Dict[str, torch.Tensor] = {"tok_embd": get("token_embd.weight"), "output_norm": get("output_norm.weight")}
    if has("output.weight"):
        w["output"] = get("output.weight")
    else:
        cfg.tie_embeddings = True
    for il, kind in enumerate(cfg.layer_kinds):
        p, b = f"l{il}", f"blk.{il}"
        if kind in ("ffn", "moe"):
            # a file may mix dense and routed FFN blocks: the router tensor tells them apart
            kind = cfg.layer_kinds[il] = "moe" if has(f"{b}.ffn_gate_inp.weight") else "ffn"
            if kind == "ffn":
                cfg.dense_ff = int(get(f"{b}.ffn_down.weight").shape[1])
        w[f"{p}.attn_norm"] = get(f"{b}.attn_norm.weight")
        for ours, theirs in _NEMOTRON_TENSORS[kind]:
            if has(f"{b}.{theirs}"):
                t = get(f"{b}.{theirs}")
                w[f"{p}.{ours}"] = t.reshape(-1) if ours in ("ssm.A", "ssm.D", "ssm.norm") else t
        if kind == "mamba2" and f"{p}.ssm.conv_b" not in w:
            w[f"{p}.ssm.conv_b"] = torch.zeros(w[f"{p}.ssm.conv_w"].shape[0])
        if kind == "nope":
            # the converter permutes q and k rows inside each head as for a rotary model; without a rotary
            # embedding the same permutation on both leaves every score unchanged, so the rows are used as stored
            w[f"{p}.attn.qkv"] = torch.cat([get(f"{b}.attn_q.weight"), get(f"{b}.attn_k.weight"),
                                            get(f"{b}.attn_v.weight")], dim=0)
        if kind == "moe":
            cfg.expert_ff = int(w[f"{p}.moe.down"].shape[2])
            cfg.shared_ff = w[f"{p}.moe.sh_down"].shape[1] if f"{p}.moe.sh_down" in w else 0
            cfg.moe_latent = w[f"{p}.moe.lat_down"].shape[0] if f"{p}.moe.lat_down" in w else 0
    return w


def config_from_gguf(md: dict) -> ModelConfig:
    a = md["general.architecture"]
    if a == "gemma4":
        return _gemma4_config(md)
    if a in ("nemotron_h", "nemotron_h_moe"):
        return _nemotron_config(md, a)
    g = lambda k, d=None: md.get(f"{a}.{k}", d)
    n_layer = int(g("block_count"))
    n_head = int(g("attention.head_count"))
    hidden = int(g("embedding_length"))
    head_dim = int(g("attention.key_length", hidden // n_head))
    kw = dict(arch=GGUF_TO_ARCH.get(a, a), n_layer=n_layer, hidden=hidden, n_head=n_head,
              n_kv_head=int(g("attention.head_count_kv", n_head)), head_dim=head_dim,
              rope_theta=float(g("rope.freq_base", 10000.0)), rope_dim=int(g("rope.dimension_count", head_dim)),
              rms_eps=float(g("attention.layer_norm_rms_epsilon", 1e-6)), vocab=int(g("vocab_size", 0)) or None,
              max_position=int(g("context_length", 131072)), n_expert=int(g("expert_count", 0)),
              top_k=int(g("expert_used_count", 0)), expert_ff=int(g("expert_feed_forward_length", 0)),
              shared_ff=int(g("expert_shared_feed_forward_length", 0)), dense_ff=int(g("feed_forward_length", 0)),
              mtp_layers=int(g("nextn_predict_layers", 0)))
    if a in ("qwen35", "qwen35moe"):
        kw.update(full_attention_interval=int(g("full_attention_interval", 4)), gated_attn=True,
                  gdn_conv=int(g("ssm.conv_kernel", 4)), gdn_k_dim=int(g("ssm.state_size", 128)),
                  gdn_k_heads=int(g("ssm.group_count", 16)), gdn_v_heads=int(g("ssm.time_step_rank", 32)),
                  gdn_tiled_heads=True, shared_gate=kw["shared_ff"] > 0)
        inner = int(g("ssm.inner_size", kw["gdn_v_heads"] * 128))
        kw["gdn_v_dim"] = inner // kw["gdn_v_heads"]
    if kw["vocab"] is None:
        kw["vocab"] = len(md.get("tokenizer.ggml.tokens", [])) or 0
    sc_kind = g("rope.scaling.type")
    if sc_kind in ("linear", "yarn") and float(g("rope.scaling.factor", 1.0)) != 1.0:
        kw["rope_scaling"] = {"type": sc_kind, "factor": float(g("rope.scaling.factor")),
                              "original_max_position_embeddings": int(g("rope.scaling.original_context_length",
                                                                        kw["max_position"]))}
    if a == "deepseek2":
        kw.update(q_lora=int(g("attention.q_lora_rank", 0)), kv_lora=int(g("attention.kv_lora_rank", 0)),
                  qk_rope_dim=int(g("rope.dimension_count", 64)), v_head_dim=int(g("attention.value_length", 128)),
                  first_dense_layers=int(g("leading_dense_block_count", 0)), qk_norm=False,
                  router_mode="sigmoid" if int(g("expert_gating_func", 2)) == 2 else "softmax",
                  route_scale=float(g("expert_weights_scale", 1.0)), n_group=int(g("expert_group_count", 1)),
                  topk_group=int(g("expert_group_used_count", 1)), router_bias=True)
        kw["qk_nope_dim"] = head_dim - kw["qk_rope_dim"]
        sc = kw.get("rope_scaling")
        if sc and sc["type"] == "yarn" and g("rope.scaling.yarn_log_multiplier") is not None:
            # this family's YaRN: cos / sin stay unscaled, the softmax scale takes the square of
            # 1 + multiplier * ln(factor)
            import math
            m = 1.0 + float(g("rope.scaling.yarn_log_multiplier")) * math.log(sc["factor"])
            sc["attention_factor"] = 1.0
            kw["attn_scale"] = head_dim ** -0.5 * m * m
    return ModelConfig(**kw)


def _gemma4_metadata(cfg: ModelConfig) -> Dict[str, object]:
    a = "gemma4"
    md = {f"{a}.block_count": cfg.n_layer, f"{a}.embedding_length": cfg.hidden, f"{a}.attention.head_count": cfg.n_head,
          f"{a}.attention.head_count_kv": [cfg.attn_dims(il)[1] for il in range(cfg.n_layer)],
          f"{a}.attention.sliding_window_pattern": [k == "swa" for k in cfg.layer_kinds],
          f"{a}.feed_forward_length": [cfg.dense_ff] * cfg.n_layer,
          f"{a}.attention.key_length": cfg.head_dim, f"{a}.attention.value_length": cfg.head_dim,
          f"{a}.attention.key_length_swa": cfg.swa_head_dim or cfg.head_dim,
          f"{a}.attention.value_length_swa": cfg.swa_head_dim or cfg.head_dim,
          f"{a}.attention.sliding_window": cfg.sliding_window, f"{a}.attention.shared_kv_layers": cfg.kv_shared_layers,
          f"{a}.rope.dimension_count": cfg.rope_dim, f"{a}.rope.freq_base": float(cfg.rope_theta),
          f"{a}.rope.freq_base_swa": float(cfg.rope_theta_swa or cfg.rope_theta),
          f"{a}.attention.layer_norm_rms_epsilon": float(cfg.rms_eps), f"{a}.context_length": cfg.max_position,
          f"{a}.final_logit_softcapping": float(cfg.logit_softcap),
          f"{a}.embedding_length_per_layer_input": cfg.ple_dim, f"{a}.vocab_size": cfg.vocab}
    if cfg.n_expert:
        md.update({f"{a}.expert_count": cfg.n_expert, f"{a}.expert_used_count": cfg.top_k,
                   f"{a}.expert_feed_forward_length": cfg.expert_ff})
    return md


def _gemma4_to_gguf(cfg: ModelConfig, w: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {"token_embd.weight": w["tok_embd"], "output_norm.weight": w["output_norm"]}
    if cfg.rope_freq_factors:
        out["rope_freqs.weight"] = torch.tensor(cfg.rope_freq_factors, dtype=torch.float32)
    if cfg.ple_dim:
        out["per_layer_token_embd.weight"] = w["ple_embd"]
        out["per_layer_model_proj.weight"] = w["ple_model_proj"]
        out["per_layer_proj_norm.weight"] = w["ple_proj_norm"]
    for il in range(cfg.n_layer):
        p, b = f"l{il}", f"blk.{il}"
        D, n_kv = cfg.attn_dims(il)
        qkv = w[f"{p}.attn.qkv"]
        nq = cfg.n_head * D
        out[f"{b}.attn_q.weight"] = qkv[:nq]
        if cfg.owns_kv(il):
            out[f"{b}.attn_k.weight"] = qkv[nq:nq + n_kv * D]
            if cfg.has_v_proj(il):
                out[f"{b}.attn_v.weight"] = qkv[nq + n_kv * D:]
            out[f"{b}.attn_k_norm.weight"] = w[f"{p}.attn.k_norm"]
        out[f"{b}.attn_q_norm.weight"] = w[f"{p}.attn.q_norm"]
        out[f"{b}.attn_output.weight"] = w[f"{p}.attn.o"]
        for ours, theirs in (("attn_norm", "attn_norm"), ("attn_post_norm", "post_attention_norm"), ("ffn_norm", "ffn_norm"),
                             ("ffn_post_norm", "post_ffw_norm"), ("ffn_post1_norm", "post_ffw_norm_1"),
                             ("ffn_pre2_norm", "pre_ffw_norm_2"), ("ffn_post2_norm", "post_ffw_norm_2"),
                             ("ple.post_norm", "post_norm")):
            if f"{p}.{ours}" in w:
                out[f"{b}.{theirs}.weight"] = w[f"{p}.{ours}"]
        F = w[f"{p}.mlp.gate_up"].shape[0] // 2       # layers that share KV may be twice as wide
        out[f"{b}.ffn_gate.weight"], out[f"{b}.ffn_up.weight"] = w[f"{p}.mlp.gate_up"][:F], w[f"{p}.mlp.gate_up"][F:]
        out[f"{b}.ffn_down.weight"] = w[f"{p}.mlp.down"]
        if cfg.is_moe_layer(il):
            out[f"{b}.ffn_gate_inp.weight"] = w[f"{p}.moe.router"]
            out[f"{b}.ffn_gate_inp.scale"] = w[f"{p}.moe.router_scale"]
            out[f"{b}.ffn_gate_up_exps.weight"] = w[f"{p}.moe.gate_up"]
            out[f"{b}.ffn_down_exps.weight"] = w[f"{p}.moe.down"]
        if cfg.layer_out_scale:
            out[f"{b}.layer_output_scale.weight"] = w[f"{p}.out_scale"]
        if cfg.ple_dim:
            out[f"{b}.inp_gate.weight"] = w[f"{p}.ple.inp_gate"]
            out[f"{b}.proj.weight"] = w[f"{p}.ple.proj"]
    return out


def _gemma4_from_gguf(cfg: ModelConfig, get, has) -> Dict[str, torch.Tensor]:
    w: Dict[str, torch.Tensor] = {"tok_embd": get("token_embd.weight"), "output_norm": get("output_norm.weight")}
    if has("rope_freqs.weight"):
        cfg.rope_freq_factors = [float(v) for v in get("rope_freqs.weight").float().reshape(-1).tolist()]
    if cfg.ple_dim:
        w["ple_embd"] = get("per_layer_token_embd.weight")
        w["ple_model_proj"] = get("per_layer_model_proj.weight")
        w["ple_proj_norm"] = get("per_layer_proj_norm.weight")
    cfg.global_k_as_v = any(not has(f"blk.{il}.attn_v.weight") for il in range(cfg.n_layer)
                            if cfg.layer_kinds[il] != "swa" and cfg.owns_kv(il))
    cfg.layer_out_scale = has("blk.0.layer_output_scale.weight")
    first_moe = next((il for il in range(cfg.n_layer) if has(f"blk.{il}.ffn_gate_inp.weight")), None)
    if first_moe is None:
        cfg.n_expert = cfg.top_k = 0
    else:
        cfg.first_dense_layers = first_moe
    for il in range(cfg.n_layer):
        p, b = f"l{il}", f"blk.{il}"
        parts = [get(f"{b}.attn_q.weight")]
        if cfg.owns_kv(il):
            parts.append(get(f"{b}.attn_k.weight"))
            if has(f"{b}.attn_v.weight"):
                parts.append(get(f"{b}.attn_v.weight"))
            w[f"{p}.attn.k_norm"] = get(f"{b}.attn_k_norm.weight")
        w[f"{p}.attn.qkv"] = torch.cat(parts, dim=0)
        w[f"{p}.attn.q_norm"] = get(f"{b}.attn_q_norm.weight")
        w[f"{p}.attn.o"] = get(f"{b}.attn_output.weight")
        for ours, theirs in (("attn_norm", "attn_norm"), ("attn_post_norm", "post_attention_norm"), ("ffn_norm", "ffn_norm"),
                             ("ffn_post_norm", "post_ffw_norm"), ("ffn_post1_norm", "post_ffw_norm_1"),
                             ("ffn_pre2_norm", "pre_ffw_norm_2"), ("ffn_post2_norm", "post_ffw_norm_2"),
                             ("ple.post_norm", "post_norm")):
            if has(f"{b}.{theirs}.weight"):
                w[f"{p}.{ours}"] = get(f"{b}.{theirs}.weight")
        w[f"{p}.mlp.gate_up"] = torch.cat([get(f"{b}.ffn_gate.weight"), get(f"{b}.ffn_up.weight")], dim=0)
        w[f"{p}.mlp.down"] = get(f"{b}.ffn_down.weight")
        if has(f"{b}.ffn_gate_inp.weight"):
            w[f"{p}.moe.router"] = get(f"{b}.ffn_gate_inp.weight")
            w[f"{p}.moe.router_scale"] = get(f"{b}.ffn_gate_inp.scale")
            if has(f"{b}.ffn_gate_up_exps.weight"):
                w[f"{p}.moe.gate_up"] = get(f"{b}.ffn_gate_up_exps.weight")
            else:
                w[f"{p}.moe.gate_up"] = torch.cat([get(f"{b}.ffn_gate_exps.weight"), get(f"{b}.ffn_up_exps.weight")], dim=1)
            w[f"{p}.moe.down"] = get(f"{b}.ffn_down_exps.weight")
        if has(f"{b}.layer_output_scale.weight"):
            w[f"{p}.out_scale"] = get(f"{b}.layer_output_scale.weight").reshape(1)
        if cfg.ple_dim:
            w[f"{p}.ple.inp_gate"] = get(f"{b}.inp_gate.weight")
            w[f"{p}.ple.proj"] = get(f"{b}.proj.weight")
    return w


def metadata_from_config(cfg: ModelConfig) -> Dict[str, object]:
    if cfg.sandwich_norm:
        return _gemma4_metadata(cfg)
    if cfg.block_form:
        return _nemotron_metadata(cfg)
    a = ARCH_TO_GGUF.get(cfg.arch, cfg.arch)
    md = {f"{a}.block_count": cfg.n_layer, f"{a}.embedding_length": cfg.hidden, f"{a}.attention.head_count": cfg.n_head,
          f"{a}.attention.head_count_kv": cfg.n_kv_head, f"{a}.attention.key_length": cfg.head_dim,
          f"{a}.attention.value_length": cfg.head_dim, f"{a}.rope.dimension_count": cfg.rope_dim,
          f"{a}.rope.freq_base": float(cfg.rope_theta), f"{a}.context_length": cfg.max_position,
          f"{a}.attention.layer_norm_rms_epsilon": float(cfg.rms_eps), f"{a}.vocab_size": cfg.vocab}
    if cfg.n_expert:
        md.update({f"{a}.expert_count": cfg.n_expert, f"{a}.expert_used_count": cfg.top_k,
                   f"{a}.expert_feed_forward_length": cfg.expert_ff})
        if cfg.shared_ff:
            md[f"{a}.expert_shared_feed_forward_length"] = cfg.shared_ff
    if cfg.dense_ff:
        md[f"{a}.feed_forward_length"] = cfg.dense_ff
    if cfg.full_attention_interval:
        md.update({f"{a}.full_attention_interval": cfg.full_attention_interval, f"{a}.ssm.conv_kernel": cfg.gdn_conv,
                   f"{a}.ssm.state_size": cfg.gdn_k_dim, f"{a}.ssm.group_count": cfg.gdn_k_heads,
                   f"{a}.ssm.time_step_rank": cfg.gdn_v_heads, f"{a}.ssm.inner_size": cfg.gdn_v_heads * cfg.gdn_v_dim})
    if cfg.mtp_layers:
        md[f"{a}.nextn_predict_layers"] = cfg.mtp_layers
    return md


# ---------------------------------------------------------------------------------------------------
# tensors
# ---------------------------------------------------------------------------------------------------
def _interleave_q_gate(q: torch.Tensor, gate: torch.Tensor, n_head: int, d: int) -> torch.Tensor:
    """[q rows | gate rows] per head, the layout of ``attn_q`` for gated attention."""
    H = q.shape[1]
    return torch.stack([q.view(n_head, d, H), gate.view(n_head, d, H)], dim=1).reshape(2 * n_head * d, H)


def to_gguf_tensors(cfg: ModelConfig, w: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    if cfg.sandwich_norm:
        return _gemma4_to_gguf(cfg, w)
    if cfg.block_form:
        return _nemotron_to_gguf(cfg, w)
    return _to_gguf_tensors(cfg, w)


def _to_gguf_tensors(cfg: ModelConfig, w: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Canonical weights -> GGUF names (splitting fused projections)."""
    out: Dict[str, torch.Tensor] = {"token_embd.weight": w["tok_embd"], "output_norm.weight": w["output_norm"]}
    if "output" in w:
        out["output.weight"] = w["output"]
    D = cfg.head_dim

    def layer(p: str, b: str, kind: str, moe: bool):
        out[f"{b}.attn_norm.weight"] = w[f"{p}.attn_norm"]
        # the norm in front of the FFN: ``post_attention_norm`` in the hybrid family's files, ``ffn_norm`` elsewhere
        ffn_norm = "post_attention_norm" if cfg.arch in ("qwen35", "qwen35moe") else "ffn_norm"
        out[f"{b}.{ffn_norm}.weight"] = w[f"{p}.ffn_norm"]
        if kind in ("attn", "swa", "nope"):
            qkv = w[f"{p}.attn.qkv"]
            qw = cfg.n_head * D * (2 if cfg.gated_attn else 1)
            out[f"{b}.attn_q.weight"] = qkv[:qw]            # already [q | gate] per head
            out[f"{b}.attn_k.weight"] = qkv[qw:qw + cfg.n_kv_head * D]
            out[f"{b}.attn_v.weight"] = qkv[qw + cfg.n_kv_head * D:]
            if cfg.qk_norm:
                out[f"{b}.attn_q_norm.weight"] = w[f"{p}.attn.q_norm"]
                out[f"{b}.attn_k_norm.weight"] = w[f"{p}.attn.k_norm"]
            out[f"{b}.attn_output.weight"] = w[f"{p}.attn.o"]
        elif kind == "gdn":
            nv = cfg.gdn_v_heads
            out[f"{b}.attn_qkv.weight"] = w[f"{p}.gdn.in_qkv"]
            out[f"{b}.attn_gate.weight"] = w[f"{p}.gdn.in_z"]
            out[f"{b}.ssm_beta.weight"] = w[f"{p}.gdn.in_ba"][:nv]
            out[f"{b}.ssm_alpha.weight"] = w[f"{p}.gdn.in_ba"][nv:]
            out[f"{b}.ssm_conv1d.weight"] = w[f"{p}.gdn.conv_w"]
            out[f"{b}.ssm_dt.bias"] = w[f"{p}.gdn.dt_bias"]
            out[f"{b}.ssm_a"] = w[f"{p}.gdn.A"]
            out[f"{b}.ssm_norm.weight"] = w[f"{p}.gdn.norm"]
            out[f"{b}.ssm_out.weight"] = w[f"{p}.gdn.out"]
        elif kind == "mla":
            for ours, theirs in (("q_a", "attn_q_a"), ("q_a_norm", "attn_q_a_norm"), ("q_b", "attn_q_b"), ("q", "attn_q"),
                                 ("kv_a", "attn_kv_a_mqa"), ("kv_a_norm", "attn_kv_a_norm"), ("kv_b", "attn_kv_b"),
                                 ("o", "attn_output")):
                if f"{p}.mla.{ours}" in w:
                    out[f"{b}.{theirs}.weight"] = w[f"{p}.mla.{ours}"]
        if moe:
            F = cfg.expert_ff
            out[f"{b}.ffn_gate_inp.weight"] = w[f"{p}.moe.router"]
            if f"{p}.moe.router_bias" in w:
                out[f"{b}.exp_probs_b.bias"] = w[f"{p}.moe.router_bias"]
            out[f"{b}.ffn_gate_exps.weight"] = w[f"{p}.moe.gate_up"][:, :F]
            out[f"{b}.ffn_up_exps.weight"] = w[f"{p}.moe.gate_up"][:, F:]
            out[f"{b}.ffn_down_exps.weight"] = w[f"{p}.moe.down"]
            if cfg.shared_ff:
                Fs = cfg.shared_ff
                out[f"{b}.ffn_gate_shexp.weight"] = w[f"{p}.moe.sh_gate_up"][:Fs]
                out[f"{b}.ffn_up_shexp.weight"] = w[f"{p}.moe.sh_gate_up"][Fs:]
                out[f"{b}.ffn_down_shexp.weight"] = w[f"{p}.moe.sh_down"]
                if cfg.shared_gate:
                    out[f"{b}.ffn_gate_inp_shexp.weight"] = w[f"{p}.moe.sh_gate"]
        elif f"{p}.mlp.gate_up" in w:
            F = cfg.dense_ff
            out[f"{b}.ffn_gate.weight"] = w[f"{p}.mlp.gate_up"][:F]
            out[f"{b}.ffn_up.weight"] = w[f"{p}.mlp.gate_up"][F:]
            out[f"{b}.ffn_down.weight"] = w[f"{p}.mlp.down"]

    for il in range(cfg.n_layer):
        layer(f"l{il}", f"blk.{il}", cfg.layer_kinds[il], cfg.is_moe_layer(il))
    for j in range(cfg.mtp_layers):
        b = f"blk.{cfg.n_layer + j}"
        p = f"mtp{j}"
        for leaf in ("eh_proj", "enorm", "hnorm", "shared_head_norm"):
            out[f"{b}.nextn.{leaf}.weight"] = w[f"{p}.{leaf}"]
        layer(f"{p}.l", b, "mla" if cfg.kv_lora > 0 else "attn", cfg.n_expert > 0)
    return {k: v.contiguous() for k, v in out.items()}


def from_gguf_tensors(cfg: ModelConfig, get, has) -> Dict[str, torch.Tensor]:
    """GGUF tensors (``get(name) -> tensor``) -> canonical fused weights."""
    if cfg.sandwich_norm:
        return _gemma4_from_gguf(cfg, get, has)
    if cfg.block_form:
        return _nemotron_from_gguf(cfg, get, has)
    w: Dict[str, torch.Tensor] = {"tok_embd": get("token_embd.weight"), "output_norm": get("output_norm.weight")}
    if has("output.weight"):
        w["output"] = get("output.weight")
    elif not cfg.tie_embeddings:
        cfg.tie_embeddings = True

    def layer(p: str, b: str, kind: str, moe: bool):
        w[f"{p}.attn_norm"] = get(f"{b}.attn_norm.weight")
        w[f"{p}.ffn_norm"] = get(f"{b}.post_attention_norm.weight") if has(f"{b}.post_attention_norm.weight") \
            else get(f"{b}.ffn_norm.weight")
        if kind in ("attn", "swa", "nope"):
            w[f"{p}.attn.qkv"] = torch.cat([get(f"{b}.attn_q.weight"), get(f"{b}.attn_k.weight"),
                                            get(f"{b}.attn_v.weight")], dim=0)
            if has(f"{b}.attn_q_norm.weight"):
                w[f"{p}.attn.q_norm"] = get(f"{b}.attn_q_norm.weight")
                w[f"{p}.attn.k_norm"] = get(f"{b}.attn_k_norm.weight")
            w[f"{p}.attn.o"] = get(f"{b}.attn_output.weight")
        elif kind == "gdn":
            w[f"{p}.gdn.in_qkv"] = get(f"{b}.attn_qkv.weight")
            w[f"{p}.gdn.in_z"] = get(f"{b}.attn_gate.weight")
            w[f"{p}.gdn.in_ba"] = torch.cat([get(f"{b}.ssm_beta.weight"), get(f"{b}.ssm_alpha.weight")], dim=0)
            cw = get(f"{b}.ssm_conv1d.weight")
            w[f"{p}.gdn.conv_w"] = cw if cw.shape[0] == cfg.gdn_conv_channels() else cw.t().contiguous()
            w[f"{p}.gdn.dt_bias"] = get(f"{b}.ssm_dt.bias")
            w[f"{p}.gdn.A"] = get(f"{b}.ssm_a").reshape(-1)
            w[f"{p}.gdn.norm"] = get(f"{b}.ssm_norm.weight")
            w[f"{p}.gdn.out"] = get(f"{b}.ssm_out.weight")
        elif kind == "mla":
            for ours, theirs in (("q_a", "attn_q_a"), ("q_a_norm", "attn_q_a_norm"), ("q_b", "attn_q_b"), ("q", "attn_q"),
                                 ("kv_a", "attn_kv_a_mqa"), ("kv_a_norm", "attn_kv_a_norm"), ("kv_b", "attn_kv_b"),
                                 ("o", "attn_output")):
                if has(f"{b}.{theirs}.weight"):
                    w[f"{p}.mla.{ours}"] = get(f"{b}.{theirs}.weight")
        if moe:
            w[f"{p}.moe.router"] = get(f"{b}.ffn_gate_inp.weight")
            if has(f"{b}.exp_probs_b.bias"):
                w[f"{p}.moe.router_bias"] = get(f"{b}.exp_probs_b.bias")
            w[f"{p}.moe.gate_up"] = torch.cat([get(f"{b}.ffn_gate_exps.weight"), get(f"{b}.ffn_up_exps.weight")], dim=1)
            w[f"{p}.moe.down"] = get(f"{b}.ffn_down_exps.weight")
            if has(f"{b}.ffn_gate_shexp.weight"):
                w[f"{p}.moe.sh_gate_up"] = torch.cat([get(f"{b}.ffn_gate_shexp.weight"),
                                                      get(f"{b}.ffn_up_shexp.weight")], dim=0)
                w[f"{p}.moe.sh_down"] = get(f"{b}.ffn_down_shexp.weight")
                if has(f"{b}.ffn_gate_inp_shexp.weight"):
                    w[f"{p}.moe.sh_gate"] = get(f"{b}.ffn_gate_inp_shexp.weight").reshape(1, -1)
        elif has(f"{b}.ffn_gate.weight"):
            w[f"{p}.mlp.gate_up"] = torch.cat([get(f"{b}.ffn_gate.weight"), get(f"{b}.ffn_up.weight")], dim=0)
            w[f"{p}.mlp.down"] = get(f"{b}.ffn_down.weight")

    for il in range(cfg.n_layer):
        layer(f"l{il}", f"blk.{il}", cfg.layer_kinds[il], cfg.is_moe_layer(il))
    for j in range(cfg.mtp_layers):
        b = f"blk.{cfg.n_layer + j}"
        p = f"mtp{j}"
        if not has(f"{b}.nextn.eh_proj.weight"):
            cfg.mtp_layers = j
            break
        for leaf in ("eh_proj", "enorm", "hnorm", "shared_head_norm"):
            w[f"{p}.{leaf}"] = get(f"{b}.nextn.{leaf}.weight")
        layer(f"{p}.l", b, "mla" if cfg.kv_lora > 0 else "attn", cfg.n_expert > 0)
    return w


def write_gguf(path: str, cfg: ModelConfig, weights: Dict[str, torch.Tensor], tokenizer=None, dtype: str = "F32",
               extra_metadata: Optional[dict] = None):
    wr = GgufWriter(path, _nemotron_arch(cfg) if cfg.block_form else ARCH_TO_GGUF.get(cfg.arch, cfg.arch))
    wr.add("general.name", f"legion-b200 {cfg.arch}")
    for k, v in metadata_from_config(cfg).items():
        wr.add(k, v)
    if tokenizer is not None and hasattr(tokenizer, "tokens"):
        wr.add("tokenizer.ggml.model", "gpt2")
        wr.add("tokenizer.ggml.tokens", list(tokenizer.tokens))
        if getattr(tokenizer, "chat_template", None):
            wr.add("tokenizer.chat_template", tokenizer.chat_template)
    for k, v in (extra_metadata or {}).items():
        wr.add(k, v)
    for name, t in to_gguf_tensors(cfg, weights).items():
        leaf_fp32 = t.dim() == 1 or name.endswith(("ssm_conv1d.weight", "ssm_a", "ssm_d", "ssm_dt.bias", "ssm_norm.weight"))
        wr.add_tensor(name, t.detach().cpu(), "F32" if leaf_fp32 else dtype)
    wr.write()


def load_gguf(path: str, device="cpu", dtype=torch.float32):
    """Returns (config, canonical weights on ``device``, metadata)."""
    gf = GgufFile(path)
    cfg = config_from_gguf(gf.metadata)
    has = lambda n: n in gf.tensors
    get = lambda n: gf.torch(n, device=device if torch.device(device).type == "cuda" else None)
    w = from_gguf_tensors(cfg, get, has)
    if cfg.vocab in (0, None):
        cfg.vocab = w["tok_embd"].shape[0]
    out = {}
    for k, v in w.items():
        out[k] = v.to(device=device, dtype=torch.float32 if is_fp32_weight(k) else dtype)
    md = gf.metadata
    return cfg, out, md
