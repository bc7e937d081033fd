"""Gemma 4 checkpoints in the Hugging Face layout (``model_type`` ``gemma4`` / ``gemma4_text``; the text model only).

The reference reads these by restating them as the ``gemma4`` GGUF llama.cpp's converter would write
(``src/hf/gemma4.rs`` in the reference) and loading that; the same route is taken here without a file in between:
the configuration becomes ``gemma4.*`` metadata and every tensor is looked up under its GGUF name, so one mapping
(``gguf_map``) builds the weights for both containers. What differs from a plain rename:

- the global layers' "proportional" rotary embedding turns only the first ``partial_rotary_factor`` of each head's
  frequency pairs; it is expressed as frequency factors (1 for the pairs that turn, 1e30 for the rest), the
  ``rope_freqs.weight`` tensor of the GGUF form;
- norm weights are used as they are (no ``+ 1``);
- the router's per-expert output scale (``router.per_expert_scale``) multiplies the routed expert's result, which
  is the same as scaling that expert's down projection, so it is folded into those weights here;
- ``layer_scalar`` is a buffer of the decoder layer and becomes the layer's output scale.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config import ModelConfig
from ..models.weights import is_fp32_weight

MODEL_TYPES = ("gemma4", "gemma4_text")

# GGUF leaf name -> name below ``layers.<il>.`` in the checkpoint
_LAYER_TENSORS = {
    "attn_q.weight": "self_attn.q_proj", "attn_k.weight": "self_attn.k_proj", "attn_v.weight": "self_attn.v_proj",
    "attn_output.weight": "self_attn.o_proj", "ffn_gate.weight": "mlp.gate_proj", "ffn_up.weight": "mlp.up_proj",
    "ffn_down.weight": "mlp.down_proj", "inp_gate.weight": "per_layer_input_gate", "proj.weight": "per_layer_projection",
}
_LAYER_VECTORS = {
    "attn_norm.weight": "input_layernorm.weight", "attn_q_norm.weight": "self_attn.q_norm.weight",
    "attn_k_norm.weight": "self_attn.k_norm.weight", "post_attention_norm.weight": "post_attention_layernorm.weight",
    "ffn_norm.weight": "pre_feedforward_layernorm.weight", "post_ffw_norm.weight": "post_feedforward_layernorm.weight",
    "post_norm.weight": "post_per_layer_input_norm.weight", "layer_output_scale.weight": "layer_scalar",
    "pre_ffw_norm_2.weight": "pre_feedforward_layernorm_2.weight",
    "post_ffw_norm_1.weight": "post_feedforward_layernorm_1.weight",
    "post_ffw_norm_2.weight": "post_feedforward_layernorm_2.weight",
    "ffn_gate_inp.weight": "router.proj.weight", "ffn_gate_inp.scale": "router.scale",
}
_TOP_TENSORS = {"token_embd.weight": "embed_tokens", "per_layer_token_embd.weight": "embed_tokens_per_layer",
                "per_layer_model_proj.weight": "per_layer_model_projection"}
_TOP_VECTORS = {"output_norm.weight": "norm.weight", "per_layer_proj_norm.weight": "per_layer_projection_norm.weight"}


def gguf_metadata(config: dict) -> Dict[str, object]:
    """``config.json`` -> the ``gemma4.*`` metadata ``gguf_map.config_from_gguf`` reads."""
    tc = dict(config.get("text_config") or config)
    n_layer = int(tc["num_hidden_layers"])
    types = tc.get("layer_types")
    if not types:
        types = ["sliding_attention" if (i + 1) % 6 else "full_attention" for i in range(n_layer)]
        types[-1] = "full_attention"
    if len(types) != n_layer:
        raise ValueError(f"gemma4: layer_types has {len(types)} entries, expected {n_layer}")
    swa = [t == "sliding_attention" for t in types]
    d_swa = int(tc.get("head_dim", 256))
    d_full = int(tc.get("global_head_dim") or d_swa)
    n_shared = int(tc.get("num_kv_shared_layers") or 0)
    rope = tc.get("rope_parameters") or {
        "sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
        "full_attention": {"rope_type": "proportional", "partial_rotary_factor": 0.25, "rope_theta": 1000000.0}}
    full, slid = rope.get("full_attention", rope), rope.get("sliding_attention", rope)
    kv_swa = int(tc.get("num_key_value_heads", 4))
    # the global layers have kv heads of their own only where keys double as values
    kv_full = int(tc.get("num_global_key_value_heads") or kv_swa) if tc.get("attention_k_eq_v") else kv_swa
    ff = int(tc["intermediate_size"])
    wide = bool(tc.get("use_double_wide_mlp")) and n_shared > 0
    a = "gemma4"
    md: Dict[str, object] = {
        "general.architecture": a, f"{a}.block_count": n_layer, f"{a}.embedding_length": int(tc["hidden_size"]),
        f"{a}.context_length": int(tc.get("max_position_embeddings") or 131072),
        f"{a}.feed_forward_length": [ff * (2 if wide and il >= n_layer - n_shared else 1) for il in range(n_layer)],
        f"{a}.attention.head_count": int(tc.get("num_attention_heads", 8)),
        f"{a}.attention.head_count_kv": [kv_swa if s else kv_full for s in swa],
        f"{a}.attention.sliding_window_pattern": swa, f"{a}.attention.sliding_window": int(tc.get("sliding_window", 512)),
        f"{a}.attention.key_length": d_full, f"{a}.attention.value_length": d_full,
        f"{a}.attention.key_length_swa": d_swa, f"{a}.attention.value_length_swa": d_swa,
        f"{a}.attention.shared_kv_layers": n_shared,
        f"{a}.attention.layer_norm_rms_epsilon": float(tc.get("rms_norm_eps", 1e-6)),
        f"{a}.rope.freq_base": float(full.get("rope_theta", 1000000.0)),
        f"{a}.rope.freq_base_swa": float(slid.get("rope_theta", full.get("rope_theta", 10000.0))),
        f"{a}.rope.dimension_count": d_full,
        f"{a}.rope.dimension_count_swa": int(d_swa * float(slid.get("partial_rotary_factor", 1.0))),
        f"{a}.embedding_length_per_layer_input": int(tc.get("hidden_size_per_layer_input") or 0),
        f"{a}.final_logit_softcapping": float(tc.get("final_logit_softcapping") or 0.0),
        f"{a}.vocab_size": int(tc["vocab_size"]),
    }
    if tc.get("enable_moe_block") and tc.get("num_experts"):
        md.update({f"{a}.expert_count": int(tc["num_experts"]), f"{a}.expert_used_count": int(tc["top_k_experts"]),
                   f"{a}.expert_feed_forward_length": int(tc.get("moe_intermediate_size")
                                                          or tc.get("expert_intermediate_size") or 0)})
    return md


def rope_factors(config: dict):
    """Frequency factors of the global layers' proportional rotary embedding, or None when every pair turns."""
    tc = dict(config.get("text_config") or config)
    rope = tc.get("rope_parameters") or {"full_attention": {"partial_rotary_factor": 0.25}}
    full = rope.get("full_attention", rope)
    d = int(tc.get("global_head_dim") or tc.get("head_dim", 256))
    n_rot = int(float(full.get("partial_rotary_factor", 1.0)) * d // 2)
    half = d // 2
    if n_rot >= half:
        return None
    return [1.0 if i < n_rot else 1e30 for i in range(half)]


def config_from_hf(config: dict) -> ModelConfig:
    from .gguf_map import config_from_gguf
    cfg = config_from_gguf(gguf_metadata(config))
    tc = dict(config.get("text_config") or config)
    cfg.vocab = int(tc["vocab_size"])
    cfg.tie_embeddings = True
    cfg.rope_freq_factors = rope_factors(config)
    cfg.global_k_as_v = bool(tc.get("attention_k_eq_v"))
    return cfg


def load(src, config: dict, dtype) -> "tuple[ModelConfig, Dict[str, torch.Tensor]]":
    """``src``: ``hf_map._Source`` over the checkpoint. Returns (config, canonical weights on the source's device)."""
    from .gguf_map import from_gguf_tensors
    cfg = config_from_hf(config)
    P = src.prefix
    factors = cfg.rope_freq_factors

    def locate(name: str):
        """GGUF name -> (checkpoint name, whether it goes through the de-quantising weight reader)."""
        if name == "rope_freqs.weight":
            return ("", False) if factors else None
        if name in _TOP_TENSORS:
            return P + _TOP_TENSORS[name], True
        if name in _TOP_VECTORS:
            return P + _TOP_VECTORS[name], False
        if not name.startswith("blk."):
            return None
        _, il, leaf = name.split(".", 2)
        lp = f"{P}layers.{il}."
        if leaf in _LAYER_TENSORS:
            return lp + _LAYER_TENSORS[leaf], True
        if leaf in _LAYER_VECTORS:
            return lp + _LAYER_VECTORS[leaf], False
        if leaf == "ffn_gate_up_exps.weight":
            return lp + "experts.gate_up_proj", False
        if leaf == "ffn_down_exps.weight":
            return lp + "experts.down_proj", False
        return None

    def has(name: str) -> bool:
        at = locate(name)
        if at is None:
            return False
        if at[0] == "":
            return True
        return src.has(at[0] + ".weight") if at[1] else src.ck.has(at[0])

    def get(name: str) -> torch.Tensor:
        at = locate(name)
        if at is None:
            raise KeyError(name)
        if at[0] == "":
            return torch.tensor(factors, dtype=torch.float32)
        if at[1]:
            return src.weight(at[0])
        t = src.raw(at[0]).to(src.device)
        if name.endswith("ffn_down_exps.weight"):
            scale = at[0].rsplit("experts.down_proj", 1)[0] + "router.per_expert_scale"
            if src.ck.has(scale):
                t = (t.float() * src.raw(scale).to(src.device).float().view(-1, 1, 1)).to(t.dtype)
        return t

    w = from_gguf_tensors(cfg, get, has)
    cfg.rope_freq_factors = factors
    out = {k: v.to(dtype=torch.float32 if is_fp32_weight(k) else dtype) for k, v in w.items()}
    return cfg, out
