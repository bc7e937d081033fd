"""Nemotron-H checkpoints in the Hugging Face layout (``model_type: nemotron_h``): a stack of blocks with ONE
sub-layer each (Mamba-2 mixer, attention without rotary embedding, squared-ReLU FFN, or the MoE with optional latent
projections), named ``backbone.*`` or ``model.*``.

Transforms on the way in (the reference's ``src/hf/nemotron_h.rs`` lists the same ones for its GGUF restatement):
``A_log`` becomes ``-exp(A_log)``; the depth-wise convolution ``[C, 1, k]`` drops its middle dimension; the per-expert
``up_proj`` / ``down_proj`` are kept stacked ``[experts, out, in]``; the router's ``e_score_correction_bias`` is the
selection bias. The block kinds come from ``layers_block_type`` or the older ``hybrid_override_pattern`` (``M`` Mamba,
``*`` attention, ``-`` FFN, ``E`` MoE)."""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config import ModelConfig
from ..models.weights import is_fp32_weight

MODEL_TYPES = ("nemotron_h",)
_KIND = {"mamba": "mamba2", "linear_attention": "mamba2", "attention": "nope", "full_attention": "nope", "mlp": "ffn",
         "moe": "moe", "M": "mamba2", "*": "nope", "-": "ffn", "E": "moe"}


def block_kinds(c: dict) -> List[str]:
    src = c.get("layers_block_type") or list(c.get("hybrid_override_pattern") or "")
    if not src:
        raise ValueError("nemotron_h: config.json has neither layers_block_type nor hybrid_override_pattern")
    try:
        return [_KIND[k] for k in src]
    except KeyError as e:
        raise ValueError(f"nemotron_h: unknown block kind {e.args[0]!r}") from None


def config_from_hf(c: dict) -> ModelConfig:
    kinds = block_kinds(c)
    hidden, n_head = int(c["hidden_size"]), int(c["num_attention_heads"])
    moe = "moe" in kinds
    kw = dict(arch="nemotron_h", n_layer=len(kinds), hidden=hidden, vocab=int(c["vocab_size"]), n_head=n_head,
              n_kv_head=int(c.get("num_key_value_heads") or n_head), head_dim=int(c.get("head_dim") or hidden // n_head),
              layer_kinds=kinds, block_form=True, qk_norm=False, ffn_act="relu2",
              rms_eps=float(c.get("layer_norm_epsilon", c.get("norm_eps", 1e-5))),
              tie_embeddings=bool(c.get("tie_word_embeddings", False)),
              max_position=int(c.get("max_position_embeddings", 4096)), dense_ff=int(c.get("intermediate_size", 0)),
              ssm_state=int(c["ssm_state_size"]), ssm_heads=int(c["mamba_num_heads"]),
              ssm_head_dim=int(c["mamba_head_dim"]), ssm_groups=int(c.get("n_groups", c.get("mamba_n_groups", 1))),
              ssm_conv=int(c.get("conv_kernel", c.get("mamba_d_conv", 4))))
    if moe:
        kw.update(n_expert=int(c["n_routed_experts"]), top_k=int(c["num_experts_per_tok"]),
                  expert_ff=int(c["moe_intermediate_size"]),
                  shared_ff=int(c.get("moe_shared_expert_intermediate_size") or 0) * (1 if c.get("n_shared_experts", 1) else 0),
                  moe_latent=int(c.get("moe_latent_size") or 0), router_mode="sigmoid", router_bias=True,
                  n_group=int(c.get("n_group", 1)), topk_group=int(c.get("topk_group", 1)),
                  norm_topk=bool(c.get("norm_topk_prob", True)), route_scale=float(c.get("routed_scaling_factor", 1.0)))
    return ModelConfig(**kw)


def load(src, config: dict, dtype) -> "tuple[ModelConfig, Dict[str, torch.Tensor]]":
    """``src``: ``hf_map._Source`` over the checkpoint. Returns (config, canonical weights on the source's device)."""
    cfg = config_from_hf(config)
    ck = src.ck
    P = "backbone." if any(n.startswith("backbone.") for n in ck.names()) else "model."
    w: Dict[str, torch.Tensor] = {}
    emb = next((P + n for n in ("embeddings", "embedding", "embed_tokens") if ck.has(f"{P}{n}.weight")), None)
    if emb is None:
        raise ValueError("nemotron_h: the checkpoint has no token embedding under a known name")
    w["tok_embd"] = src.weight(emb)
    w["output_norm"] = src.raw(P + "norm_f.weight").to(src.device)
    if ck.has("lm_head.weight"):
        w["output"] = src.weight("lm_head")
    else:
        cfg.tie_embeddings = True
    if cfg.tie_embeddings:
        w.pop("output", None)
    vec = lambda name: src.raw(name).to(src.device).float()        # noqa: E731
    for il, kind in enumerate(cfg.layer_kinds):
        p, lp = f"l{il}", f"{P}layers.{il}."
        m = lp + "mixer."
        w[f"{p}.attn_norm"] = vec(lp + "norm.weight")
        if kind == "mamba2":
            w[f"{p}.ssm.in"] = src.weight(m + "in_proj")
            cw = src.raw(m + "conv1d.weight").to(src.device)
            w[f"{p}.ssm.conv_w"] = cw.reshape(cw.shape[0], cw.shape[-1]).float()
            w[f"{p}.ssm.conv_b"] = (vec(m + "conv1d.bias") if ck.has(m + "conv1d.bias")
                                    else torch.zeros(cw.shape[0], device=src.device))
            w[f"{p}.ssm.A"] = -torch.exp(vec(m + "A_log"))
            w[f"{p}.ssm.D"] = vec(m + "D")
            w[f"{p}.ssm.dt_bias"] = vec(m + "dt_bias")
            w[f"{p}.ssm.norm"] = vec(m + "norm.weight")
            w[f"{p}.ssm.out"] = src.weight(m + "out_proj")
        elif kind == "nope":
            w[f"{p}.attn.qkv"] = torch.cat([src.weight(m + "q_proj"), src.weight(m + "k_proj"),
                                            src.weight(m + "v_proj")], dim=0)
            w[f"{p}.attn.o"] = src.weight(m + "o_proj")
        elif kind == "ffn":
            w[f"{p}.mlp.gate_up"] = src.weight(m + "up_proj")
            w[f"{p}.mlp.down"] = src.weight(m + "down_proj")
        else:
            w[f"{p}.moe.router"] = src.raw(m + "gate.weight").to(src.device)
            w[f"{p}.moe.router_bias"] = vec(m + "gate.e_score_correction_bias")
            if ck.has(m + "experts.up_proj"):
                w[f"{p}.moe.gate_up"] = src.raw(m + "experts.up_proj").to(src.device)
                w[f"{p}.moe.down"] = src.raw(m + "experts.down_proj").to(src.device)
            else:                                   # one module per expert
                w[f"{p}.moe.gate_up"] = torch.stack([src.weight(f"{m}experts.{e}.up_proj") for e in range(cfg.n_expert)])
                w[f"{p}.moe.down"] = torch.stack([src.weight(f"{m}experts.{e}.down_proj") for e in range(cfg.n_expert)])
            if cfg.moe_latent:
                w[f"{p}.moe.lat_down"] = src.weight(m + "fc1_latent_proj")
                w[f"{p}.moe.lat_up"] = src.weight(m + "fc2_latent_proj")
            if cfg.shared_ff:
                w[f"{p}.moe.sh_gate_up"] = src.weight(m + "shared_experts.up_proj")
                w[f"{p}.moe.sh_down"] = src.weight(m + "shared_experts.down_proj")
    out = {k: v.to(dtype=torch.float32 if is_fp32_weight(k) else dtype) for k, v in w.items()}
    return cfg, out
