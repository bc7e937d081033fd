"""HF checkpoint directories -> canonical fused weights (and back, for writing test checkpoints).

``config.json`` ``model_type`` selects the mapper: ``qwen3`` / ``qwen3_moe`` / ``llama`` / ``mistral``,
``qwen3_next`` / ``qwen3_5`` / ``qwen3_5_moe`` (hybrid Gated DeltaNet), ``deepseek_v3`` (MLA), ``gemma4`` /
``gemma4_text`` (``hf_gemma4``), ``nemotron_h`` (``hf_nemotron``).
Transforms applied while loading the Qwen3.5 family (``src/hf/qwen35.rs:6-20`` in the reference):
``A_log -> -exp(A_log)``; RMSNorm weights stored as (w - 1) get +1 (all but the DeltaNet output norm);
fused ``in_proj_qkvz`` / ``in_proj_ba`` are de-interleaved per key head; conv1d ``[C, 1, k]`` is squeezed;
experts are stacked to 3-D with gate and up concatenated; quantised tensors (FP8 per-tensor / per-channel /
128x128 blocks, NVFP4 ModelOpt / compressed-tensors) are decoded to the compute dtype.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Optional

import torch

from ..config import ModelConfig
from ..models.weights import is_fp32_weight, weight_shapes
from . import hf_gemma4, hf_nemotron
from . import quant_formats as qf
from .safetensors_io import Checkpoint, save_file

HYBRID_TYPES = ("qwen3_next", "qwen3_5", "qwen3_5_moe", "qwen3_5_text", "qwen3_5_moe_text")


def config_from_hf(c: dict) -> ModelConfig:
    if (c.get("text_config") or c).get("model_type") in hf_gemma4.MODEL_TYPES or c.get("model_type") == "gemma4":
        return hf_gemma4.config_from_hf(c)
    if c.get("model_type") in hf_nemotron.MODEL_TYPES:
        return hf_nemotron.config_from_hf(c)
    c = dict(c.get("text_config") or c)
    mt = c.get("model_type", "llama")
    n_head = c["num_attention_heads"]
    hidden = c["hidden_size"]
    kw = dict(n_layer=c["num_hidden_layers"], hidden=hidden, vocab=c["vocab_size"], n_head=n_head,
              n_kv_head=c.get("num_key_value_heads", n_head), head_dim=c.get("head_dim") or hidden // n_head,
              rope_theta=float(c.get("rope_theta", 10000.0)), rms_eps=float(c.get("rms_norm_eps", 1e-6)),
              tie_embeddings=bool(c.get("tie_word_embeddings", False)),
              max_position=int(c.get("max_position_embeddings", 131072)), rope_scaling=c.get("rope_scaling"))
    rp = c.get("rope_scaling") or c.get("rope_parameters") or {}
    if isinstance(rp, dict) and "rope_theta" in rp and "rope_theta" not in c:
        kw["rope_theta"] = float(rp["rope_theta"])
    if isinstance(rp, dict) and rp.get("rope_type", rp.get("type", "default")) not in ("default", None):
        kw["rope_scaling"] = dict(rp)         # newer configs keep the scaling beside the base in ``rope_parameters``
    if isinstance(rp, dict) and rp.get("mrope_section"):
        # vision-language checkpoints: rotary frequencies turn with (temporal, row, column) positions
        kw["mrope_sections"] = tuple(int(v) for v in rp["mrope_section"][:3])
        kw["mrope_interleaved"] = bool(rp.get("mrope_interleaved", False))
        if "rope_theta" in rp:
            kw["rope_theta"] = float(rp["rope_theta"])
    if mt in ("qwen3", "qwen3_moe", "qwen3_vl_text", "qwen3_vl_moe_text", "qwen3_vl", "qwen3_vl_moe"):
        kw.update(arch="qwen3moe" if "moe" in mt else "qwen3", qk_norm=True)
    elif mt in HYBRID_TYPES:
        moe = c.get("num_experts", 0) > 0
        kinds = c.get("layer_types")
        kw.update(arch="qwen35moe" if moe else "qwen35", qk_norm=True, gated_attn=True, norm_offset=1.0,
                  full_attention_interval=int(c.get("full_attention_interval", 4)),
                  rope_dim=int(kw["head_dim"] * float(c.get("partial_rotary_factor", 0.25))),
                  gdn_k_heads=c.get("linear_num_key_heads", 16), gdn_v_heads=c.get("linear_num_value_heads", 32),
                  gdn_k_dim=c.get("linear_key_head_dim", 128), gdn_v_dim=c.get("linear_value_head_dim", 128),
                  gdn_conv=c.get("linear_conv_kernel_dim", 4), mtp_layers=int(c.get("mtp_num_hidden_layers", 0) or 0))
        if kinds:
            kw["layer_kinds"] = ["gdn" if k == "linear_attention" else "attn" for k in kinds]
            kw["full_attention_interval"] = 0
    elif mt in ("deepseek_v3", "deepseek_v2", "kimi_k2"):
        kw.update(arch="deepseek_v3", qk_norm=False, q_lora=c.get("q_lora_rank") or 0, kv_lora=c["kv_lora_rank"],
                  qk_nope_dim=c["qk_nope_head_dim"], qk_rope_dim=c["qk_rope_head_dim"], v_head_dim=c["v_head_dim"],
                  head_dim=c["qk_nope_head_dim"] + c["qk_rope_head_dim"], dense_ff=c["intermediate_size"],
                  first_dense_layers=c.get("first_k_dense_replace", 0), n_expert=c.get("n_routed_experts", 0),
                  top_k=c.get("num_experts_per_tok", 0), expert_ff=c.get("moe_intermediate_size", 0),
                  shared_ff=c.get("moe_intermediate_size", 0) * c.get("n_shared_experts", 0),
                  router_mode="sigmoid" if c.get("scoring_func", "sigmoid") == "sigmoid" else "softmax",
                  router_bias=c.get("topk_method", "noaux_tc") == "noaux_tc", n_group=c.get("n_group", 1),
                  topk_group=c.get("topk_group", 1), route_scale=float(c.get("routed_scaling_factor", 1.0)),
                  norm_topk=bool(c.get("norm_topk_prob", True)), mtp_layers=int(c.get("num_nextn_predict_layers", 0)))
        sc = kw.get("rope_scaling") or {}
        if sc.get("rope_type", sc.get("type")) == "yarn" and sc.get("mscale_all_dim"):
            # this family also scales the softmax by the square of the all-dimension YaRN term
            from ..ops.reference import yarn_mscale
            m = yarn_mscale(float(sc.get("factor", 1.0)), float(sc["mscale_all_dim"]))
            kw["attn_scale"] = (c["qk_nope_head_dim"] + c["qk_rope_head_dim"]) ** -0.5 * m * m
    else:
        kw.update(arch="llama" if mt in ("llama", "mistral") else mt, qk_norm=False)
    if mt not in ("deepseek_v3", "deepseek_v2", "kimi_k2"):
        ne = c.get("num_experts", c.get("num_local_experts", 0)) or 0
        if ne:
            kw.update(n_expert=ne, top_k=c.get("num_experts_per_tok", 2),
                      expert_ff=c.get("moe_intermediate_size", c.get("intermediate_size")),
                      norm_topk=bool(c.get("norm_topk_prob", True)),
                      shared_ff=c.get("shared_expert_intermediate_size", 0) or 0)
            kw["shared_gate"] = kw["shared_ff"] > 0
            dense = sorted(int(i) for i in (c.get("mlp_only_layers") or []))
            if dense or int(c.get("decoder_sparse_step", 1) or 1) != 1:
                # dense layers are modelled as a leading run only
                if dense != list(range(len(dense))) or int(c.get("decoder_sparse_step", 1) or 1) != 1:
                    raise ValueError("dense FFN layers between MoE layers (mlp_only_layers / decoder_sparse_step) are "
                                     "supported only as a leading run")
                kw["first_dense_layers"] = len(dense)
                kw["dense_ff"] = c["intermediate_size"]
        else:
            kw["dense_ff"] = c["intermediate_size"]
    return ModelConfig(**kw)


class _Source:
    """Tensor access with on-the-fly de-quantisation of FP8 / NVFP4 weights."""

    def __init__(self, ck: Checkpoint, device, dtype):
        self.ck, self.device, self.dtype = ck, device, dtype
        self.method = ck.quant_method()
        self.prefix = ""
        for cand in ("model.language_model.", "language_model.model.", "model."):
            if any(n.startswith(cand + "layers.") for n in ck.names()):
                self.prefix = cand
                break

    def has(self, name: str) -> bool:
        return self.ck.has(name) or self.ck.has(name + "_packed")

    def raw(self, name: str) -> torch.Tensor:
        return self.ck.get(name)

    def shipped(self, base: str):
        """The tensor's quantised parts exactly as the checkpoint stores them, on the device, or None when it is
        not block-quantised: ("nvfp4", codes u8 [rows, K/2], scale bytes u8 [rows, K/16], tensor scale) or
        ("fp8", e4m3 bytes u8 [rows, K], fp32 scale per 128 x 128 block)."""
        ck, dev = self.ck, self.device
        if ck.has(base + ".weight_packed"):                       # compressed-tensors NVFP4: the global scale divides
            g = 1.0 / float(ck.get(base + ".weight_global_scale").float().reshape(-1)[0])
            return ("nvfp4", ck.get(base + ".weight_packed").to(dev).view(torch.uint8),
                    ck.get(base + ".weight_scale").view(torch.uint8).to(dev), g)
        if not ck.has(base + ".weight"):
            return None
        if ck.has(base + ".weight_scale_2"):                      # ModelOpt NVFP4
            return ("nvfp4", ck.get(base + ".weight").to(dev).view(torch.uint8),
                    ck.get(base + ".weight_scale").view(torch.uint8).to(dev),
                    float(ck.get(base + ".weight_scale_2").float().reshape(-1)[0]))
        w = ck.get(base + ".weight")
        if w.dtype == torch.float8_e4m3fn and ck.has(base + ".weight_scale_inv"):
            bs = (ck.config.get("quantization_config") or {}).get("weight_block_size") or [128, 128]
            if list(bs) == [128, 128]:
                return ("fp8", w.view(torch.uint8).to(dev), ck.get(base + ".weight_scale_inv").float().to(dev))
        return None

    def stacked(self, bases, dual: bool = False, groups: int = 1):
        """Several checkpoint tensors stacked by rows WITHOUT leaving their encoding: ``bases`` lists, group by
        group, the tensors of each group in row order (``dual``: two per group, the gate and the up half, each with
        its own tensor scale). Returns an ``ops.sm100.Nv4Weight`` / ``Fp8Weight`` ([groups, rows, K] when groups > 1)
        or None when a part is not quantised, the parts differ in kind, or the shapes do not fit the kernels."""
        from ..ops import sm100
        if self.device.type != "cuda":
            return None
        parts = [self.shipped(b) for b in bases]
        if any(p is None for p in parts) or len({p[0] for p in parts}) != 1:
            return None
        per = len(parts) // groups
        kind = parts[0][0]
        rows = [p[1].shape[0] for p in parts]
        if any(r % 128 for r in rows):
            return None
        if kind == "nvfp4":
            K = parts[0][1].shape[1] * 2
            if K % 64:
                return None
            gs = [p[3] for p in parts]
            if not dual and per > 1 and len(set(gs[:per])) > 1:
                return None                        # one tensor scale per group: parts of a group must share it
            codes = torch.cat([p[1] for p in parts], 0)
            scales = torch.cat([p[2] for p in parts], 0)
            g = torch.tensor(gs if dual else gs[::per], dtype=torch.float32, device=self.device)
            if groups > 1:
                codes = codes.view(groups, -1, codes.shape[-1])
                scales = scales.view(groups, -1, scales.shape[-1])
            return sm100.Nv4Weight.from_parts(codes, scales, g)
        data = torch.cat([p[1] for p in parts], 0)
        sc = torch.cat([p[2] for p in parts], 0)
        if groups > 1:
            data = data.view(groups, -1, data.shape[-1])
            sc = sc.view(groups, -1, sc.shape[-1])
        return sm100.Fp8Weight(data.contiguous(), sc.contiguous())

    def weight(self, base: str) -> torch.Tensor:
        """``base`` without the ``.weight`` suffix."""
        ck = self.ck
        dev = self.device
        if ck.has(base + ".weight_packed"):                       # compressed-tensors NVFP4
            codes = ck.get(base + ".weight_packed").to(dev)
            sc = ck.get(base + ".weight_scale").to(dev)
            g = ck.get(base + ".weight_global_scale")
            return qf.nvfp4_dequant(codes, sc, g, self.dtype, global_is_divisor=True)
        w = ck.get(base + ".weight")
        if ck.has(base + ".weight_scale_2"):                      # ModelOpt NVFP4
            return qf.nvfp4_dequant(w.to(dev), ck.get(base + ".weight_scale").to(dev), ck.get(base + ".weight_scale_2"),
                                    self.dtype)
        if w.dtype == torch.float8_e4m3fn:
            if ck.has(base + ".weight_scale_inv"):
                bs = (ck.config.get("quantization_config") or {}).get("weight_block_size") or [128, 128]
                return qf.fp8_dequant(w.to(dev), ck.get(base + ".weight_scale_inv").to(dev), (bs[0], bs[1]), self.dtype)
            return qf.fp8_dequant(w.to(dev), ck.get(base + ".weight_scale").to(dev), None, self.dtype)
        return w.to(device=dev)


def load_hf(path: str, device="cpu", dtype=torch.float32, keep_quant: bool = False, expert_range=None,
            keep_quant_dense: bool = True, read_threads: int = 0):
    """Returns (config, canonical weights, checkpoint). ``keep_quant`` (CUDA device): block-quantised expert, FFN
    and output projections stay in their shipped encoding (``ops.sm100.Nv4Weight`` / ``Fp8Weight``: the file's code
    bytes, scale bytes re-ordered for the tensor-core copy, never expanded to bf16), the way the reference repacks
    ModelOpt / compressed-tensors tensors (``src/hf/nvfp4.rs:5-33``) and picks the matmul per tensor
    (``src/model/core/linear.rs:95-112``). Tensors whose rows are interleaved or permuted on the way in (fused
    attention / DeltaNet projections, rotary de-interleave) are decoded. ``expert_range=(lo, hi)``: only these
    routed experts are read (an expert-parallel rank reads its own shard of the files and nothing else of the
    experts, like the reference's sharded reader ``src/load_io.rs``). ``keep_quant_dense=False`` keeps only the
    experts encoded (ranks that slice the dense projections by columns decode those first). ``read_threads`` > 0:
    every layer's tensors (of the routed experts only those in ``expert_range``) are read ahead by that many
    threads of positional reads instead of through the memory map."""
    ck = Checkpoint(path)
    if (ck.config.get("text_config") or ck.config).get("model_type") in hf_gemma4.MODEL_TYPES \
            or ck.config.get("model_type") == "gemma4":
        cfg, w = hf_gemma4.load(_Source(ck, torch.device(device), dtype), ck.config, dtype)
        return cfg, w, ck
    if ck.config.get("model_type") in hf_nemotron.MODEL_TYPES:
        cfg, w = hf_nemotron.load(_Source(ck, torch.device(device), dtype), ck.config, dtype)
        return cfg, w, ck
    cfg = config_from_hf(ck.config)
    src = _Source(ck, torch.device(device), dtype)
    P = src.prefix
    hybrid = (ck.config.get("text_config") or ck.config).get("model_type") in HYBRID_TYPES
    w: Dict[str, torch.Tensor] = {}

    def norm(name):
        return src.raw(name).float()

    def proj(base):
        """A projection that is used as stored (no row permutation): stays encoded when asked for."""
        q = src.stacked([base]) if (keep_quant and keep_quant_dense) else None
        return q if q is not None else src.weight(base)

    w["tok_embd"] = src.weight(P + "embed_tokens")
    w["output_norm"] = norm(P + "norm.weight")
    if ck.has("lm_head.weight") or ck.has("lm_head.weight_packed"):
        w["output"] = src.weight("lm_head")
    else:
        cfg.tie_embeddings = True
    D = cfg.head_dim

    def experts(pre: str, p: str):
        e_lo, e_hi = expert_range if expert_range is not None else (0, cfg.n_expert)
        E = e_hi - e_lo
        if ck.has(pre + "experts.gate_up_proj"):                  # already fused [E, H, 2F] or [E, 2F, H]
            gu = src.raw(pre + "experts.gate_up_proj")[e_lo:e_hi]
            dn = src.raw(pre + "experts.down_proj")[e_lo:e_hi]
            # [E, H, 2F] / [E, F, H] (older exports) or [E, 2F, H] / [E, H, F]: told apart by whichever of the two
            # tensors is not square-ambiguous
            if dn.shape[1] != dn.shape[2]:
                flipped = dn.shape[2] == cfg.hidden
            else:
                flipped = gu.shape[1] == cfg.hidden and gu.shape[2] != cfg.hidden
            if flipped:
                gu, dn = gu.transpose(1, 2), dn.transpose(1, 2)
            w[f"{p}.moe.gate_up"], w[f"{p}.moe.down"] = gu.contiguous(), dn.contiguous()
            return
        if keep_quant:
            qg = src.stacked([f"{pre}experts.{e}.{n}" for e in range(e_lo, e_hi) for n in ("gate_proj", "up_proj")],
                             dual=True, groups=E)
            qd = src.stacked([f"{pre}experts.{e}.down_proj" for e in range(e_lo, e_hi)], groups=E) if qg is not None else None
            if qg is not None and qd is not None:
                w[f"{p}.moe.gate_up"], w[f"{p}.moe.down"] = qg, qd
                return
        gus, dns = [], []
        for e in range(e_lo, e_hi):
            g = src.weight(f"{pre}experts.{e}.gate_proj")
            u = src.weight(f"{pre}experts.{e}.up_proj")
            gus.append(torch.cat([g, u], dim=0))
            dns.append(src.weight(f"{pre}experts.{e}.down_proj"))
        w[f"{p}.moe.gate_up"] = torch.stack(gus)
        w[f"{p}.moe.down"] = torch.stack(dns)

    def ffn(lp: str, p: str, moe: bool):
        if moe:
            pre = lp + "mlp."
            w[f"{p}.moe.router"] = src.weight(pre + "gate")
            if ck.has(pre + "gate.e_score_correction_bias"):
                w[f"{p}.moe.router_bias"] = src.raw(pre + "gate.e_score_correction_bias").float()
            experts(pre, p)
            for sh in ("shared_expert.", "shared_experts."):
                if ck.has(pre + sh + "gate_proj.weight") or ck.has(pre + sh + "gate_proj.weight_packed"):
                    if keep_quant and keep_quant_dense:
                        qg = src.stacked([pre + sh + "gate_proj", pre + sh + "up_proj"], dual=True)
                        qd = src.stacked([pre + sh + "down_proj"]) if qg is not None else None
                        if qg is not None and qd is not None:
                            w[f"{p}.moe.sh_gate_up"], w[f"{p}.moe.sh_down"] = qg, qd
                            continue
                    w[f"{p}.moe.sh_gate_up"] = torch.cat([src.weight(pre + sh + "gate_proj"),
                                                          src.weight(pre + sh + "up_proj")], dim=0)
                    w[f"{p}.moe.sh_down"] = src.weight(pre + sh + "down_proj")
            if ck.has(pre + "shared_expert_gate.weight"):
                w[f"{p}.moe.sh_gate"] = src.weight(pre + "shared_expert_gate").reshape(1, -1)
        else:
            if keep_quant and keep_quant_dense:
                qg = src.stacked([lp + "mlp.gate_proj", lp + "mlp.up_proj"], dual=True)
                qd = src.stacked([lp + "mlp.down_proj"]) if qg is not None else None
                if qg is not None and qd is not None:
                    w[f"{p}.mlp.gate_up"], w[f"{p}.mlp.down"] = qg, qd
                    return
            w[f"{p}.mlp.gate_up"] = torch.cat([src.weight(lp + "mlp.gate_proj"), src.weight(lp + "mlp.up_proj")], dim=0)
            w[f"{p}.mlp.down"] = src.weight(lp + "mlp.down_proj")

    def attention(lp: str, p: str):
        a = lp + "self_attn."
        q = src.weight(a + "q_proj")
        w[f"{p}.attn.qkv"] = torch.cat([q, src.weight(a + "k_proj"), src.weight(a + "v_proj")], dim=0)
        if ck.has(a + "q_norm.weight"):
            w[f"{p}.attn.q_norm"] = norm(a + "q_norm.weight")
            w[f"{p}.attn.k_norm"] = norm(a + "k_norm.weight")
        w[f"{p}.attn.o"] = proj(a + "o_proj")

    def deltanet(lp: str, p: str):
        a = lp + "linear_attn."
        nk, nv, dk, dv = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_k_dim, cfg.gdn_v_dim
        r = nv // nk
        H = cfg.hidden
        if ck.has(a + "in_proj_qkvz.weight"):
            # rows are grouped per key head: [q(dk) | k(dk) | v(r*dv) | z(r*dv)]
            t = src.weight(a + "in_proj_qkvz").view(nk, 2 * dk + 2 * r * dv, H)
            q, k = t[:, :dk], t[:, dk:2 * dk]
            v, z = t[:, 2 * dk:2 * dk + r * dv], t[:, 2 * dk + r * dv:]
            w[f"{p}.gdn.in_qkv"] = torch.cat([q.reshape(-1, H), k.reshape(-1, H), v.reshape(-1, H)], dim=0)
            w[f"{p}.gdn.in_z"] = z.reshape(-1, H).contiguous()
            ba = src.weight(a + "in_proj_ba").view(nk, 2 * r, H)
            w[f"{p}.gdn.in_ba"] = torch.cat([ba[:, :r].reshape(-1, H), ba[:, r:].reshape(-1, H)], dim=0)
        else:
            w[f"{p}.gdn.in_qkv"] = src.weight(a + "in_proj_qkv")
            w[f"{p}.gdn.in_z"] = src.weight(a + "in_proj_z")
            w[f"{p}.gdn.in_ba"] = torch.cat([src.weight(a + "in_proj_b"), src.weight(a + "in_proj_a")], dim=0)
        w[f"{p}.gdn.conv_w"] = src.raw(a + "conv1d.weight").float().reshape(cfg.gdn_conv_channels(), -1)
        w[f"{p}.gdn.A"] = -torch.exp(src.raw(a + "A_log").float())
        w[f"{p}.gdn.dt_bias"] = src.raw(a + "dt_bias").float()
        w[f"{p}.gdn.norm"] = norm(a + "norm.weight")       # stored as the plain weight (no +1)
        w[f"{p}.gdn.out"] = proj(a + "out_proj")

    def mla(lp: str, p: str):
        a = lp + "self_attn."
        if cfg.q_lora:
            w[f"{p}.mla.q_a"] = src.weight(a + "q_a_proj")
            w[f"{p}.mla.q_a_norm"] = norm(a + "q_a_layernorm.weight")
            w[f"{p}.mla.q_b"] = _deinterleave_rope(src.weight(a + "q_b_proj"), cfg.n_head, cfg.qk_nope_dim, cfg.qk_rope_dim)
        else:
            w[f"{p}.mla.q"] = _deinterleave_rope(src.weight(a + "q_proj"), cfg.n_head, cfg.qk_nope_dim, cfg.qk_rope_dim)
        kva = src.weight(a + "kv_a_proj_with_mqa")
        w[f"{p}.mla.kv_a"] = _deinterleave_rope(kva, 1, cfg.kv_lora, cfg.qk_rope_dim)
        w[f"{p}.mla.kv_a_norm"] = norm(a + "kv_a_layernorm.weight")
        w[f"{p}.mla.kv_b"] = src.weight(a + "kv_b_proj")
        w[f"{p}.mla.o"] = proj(a + "o_proj")

    def read_ahead(prefix: str):
        if read_threads <= 0:
            return
        names = [n for n in ck.names() if n.startswith(prefix)]
        if expert_range is not None:
            lo, hi = expert_range
            keep = []
            for n in names:
                i = n.find(".experts.")
                if i >= 0:
                    e = n[i + 9:].split(".", 1)[0]
                    if e.isdigit() and not (lo <= int(e) < hi):
                        continue
                keep.append(n)
            names = keep
        ck.prefetch(names, threads=read_threads, pin=torch.device(device).type == "cuda")

    for il in range(cfg.n_layer):
        lp, p = f"{P}layers.{il}.", f"l{il}"
        read_ahead(lp)
        w[f"{p}.attn_norm"] = norm(lp + "input_layernorm.weight")
        w[f"{p}.ffn_norm"] = norm(lp + "post_attention_layernorm.weight")
        kind = cfg.layer_kinds[il]
        if kind == "gdn":
            deltanet(lp, p)
        elif kind == "mla":
            mla(lp, p)
        else:
            attention(lp, p)
        ffn(lp, p, cfg.is_moe_layer(il))
    # the draft head (MTP), when the checkpoint ships it: DeepSeek appends it as layer n_layer + j with the fusion
    # tensors beside the block's, the hybrid family keeps it under ``mtp.``; checkpoints without it lose the flag
    for j in range(cfg.mtp_layers):
        mp = f"mtp{j}"
        if hybrid:
            lp, names = f"mtp.layers.{j}.", ("mtp.fc", "mtp.pre_fc_norm_embedding.weight", "mtp.pre_fc_norm_hidden.weight",
                                             "mtp.norm.weight")
        else:
            lp = f"{P}layers.{cfg.n_layer + j}."
            names = (lp + "eh_proj", lp + "enorm.weight", lp + "hnorm.weight", lp + "shared_head.norm.weight")
        if not src.has(names[0] + ".weight"):
            cfg.mtp_layers = j
            break
        w[f"{mp}.eh_proj"] = src.weight(names[0])
        w[f"{mp}.enorm"], w[f"{mp}.hnorm"], w[f"{mp}.shared_head_norm"] = norm(names[1]), norm(names[2]), norm(names[3])
        w[f"{mp}.l.attn_norm"] = norm(lp + "input_layernorm.weight")
        w[f"{mp}.l.ffn_norm"] = norm(lp + "post_attention_layernorm.weight")
        (mla if cfg.kv_lora > 0 else attention)(lp, f"{mp}.l")
        ffn(lp, f"{mp}.l", cfg.n_expert > 0)
    # the engine applies ``norm_offset`` at run time, so (w - 1) checkpoints are kept as stored
    out = {}
    for k, v in w.items():
        if not isinstance(v, torch.Tensor):
            out[k] = v                          # kept in its shipped encoding
            continue
        out[k] = v.to(device=device, dtype=torch.float32 if is_fp32_weight(k) else dtype).contiguous()
    return cfg, out, ck


def _deinterleave_rope(wt: torch.Tensor, n_head: int, d_nope: int, d_rope: int) -> torch.Tensor:
    """DeepSeek checkpoints store rotary dims as interleaved (re, im) pairs; the engine's RoPE pairs
    dim i with i + d_rope/2, so the rope rows of each head are permuted [0,2,4,...,1,3,5,...]."""
    per = d_nope + d_rope
    t = wt.view(n_head, per, -1)
    idx = torch.cat([torch.arange(0, d_rope, 2), torch.arange(1, d_rope, 2)]) + d_nope
    full = torch.cat([torch.arange(d_nope), idx])
    return t[:, full].reshape(n_head * per, -1).contiguous()


# ---------------------------------------------------------------------------------------------------
# writer (test checkpoints and ``legion st`` round trips)
# ---------------------------------------------------------------------------------------------------
def save_hf(path: str, cfg: ModelConfig, w: Dict[str, torch.Tensor], quant: str = "none", dtype=torch.bfloat16):
    """Writes ``config.json`` + ``model.safetensors`` in HF naming (qwen3 / qwen3_moe / hybrid / deepseek_v3).
    ``quant``: none | fp8_block | nvfp4 (ModelOpt layout) | nvfp4_ct (compressed-tensors layout)."""
    os.makedirs(path, exist_ok=True)
    t: Dict[str, torch.Tensor] = {}

    def put(base: str, x: torch.Tensor, quantise: bool = True):
        x = x.detach().cpu()
        if quant == "none" or not quantise or x.dim() != 2 or x.shape[1] % 16:
            t[base + ".weight"] = x.to(dtype)
        elif quant == "fp8_block":
            q, s = qf.fp8_block_quant(x.float())
            t[base + ".weight"], t[base + ".weight_scale_inv"] = q, s
        elif quant == "nvfp4":
            c, s, g = qf.nvfp4_quant(x.float())
            t[base + ".weight"], t[base + ".weight_scale"], t[base + ".weight_scale_2"] = c, s, g.reshape(())
            t[base + ".input_scale"] = torch.tensor(1.0)
        elif quant == "nvfp4_ct":
            c, s, g = qf.nvfp4_quant(x.float())
            t[base + ".weight_packed"], t[base + ".weight_scale"] = c, s
            t[base + ".weight_global_scale"] = (1.0 / g).reshape(1)
        else:
            raise ValueError(quant)

    P = "model."
    put(P + "embed_tokens", w["tok_embd"], False)
    t[P + "norm.weight"] = w["output_norm"].cpu().to(dtype)
    if "output" in w:
        put("lm_head", w["output"], False)
    D = cfg.head_dim
    blocks = [(f"{P}layers.{il}.", f"l{il}", cfg.layer_kinds[il], cfg.is_moe_layer(il)) for il in range(cfg.n_layer)]
    hybrid = cfg.arch in ("qwen35", "qwen35moe")
    for j in range(cfg.mtp_layers if f"mtp0.eh_proj" in w else 0):
        # the draft head: DeepSeek appends it as layer n_layer + j, the hybrid family keeps it under ``mtp.``
        mp = f"mtp{j}"
        if hybrid:
            lp = f"mtp.layers.{j}."
            put("mtp.fc", w[f"{mp}.eh_proj"], False)
            t["mtp.pre_fc_norm_embedding.weight"] = w[f"{mp}.enorm"].cpu().to(dtype)
            t["mtp.pre_fc_norm_hidden.weight"] = w[f"{mp}.hnorm"].cpu().to(dtype)
            t["mtp.norm.weight"] = w[f"{mp}.shared_head_norm"].cpu().to(dtype)
        else:
            lp = f"{P}layers.{cfg.n_layer + j}."
            put(lp + "eh_proj", w[f"{mp}.eh_proj"], False)
            t[lp + "enorm.weight"] = w[f"{mp}.enorm"].cpu().to(dtype)
            t[lp + "hnorm.weight"] = w[f"{mp}.hnorm"].cpu().to(dtype)
            t[lp + "shared_head.norm.weight"] = w[f"{mp}.shared_head_norm"].cpu().to(dtype)
        blocks.append((lp, f"{mp}.l", "mla" if cfg.kv_lora > 0 else "attn", cfg.n_expert > 0))
    for lp, p, kind, moe_block in blocks:
        t[lp + "input_layernorm.weight"] = w[f"{p}.attn_norm"].cpu().to(dtype)
        t[lp + "post_attention_layernorm.weight"] = w[f"{p}.ffn_norm"].cpu().to(dtype)
        if kind in ("attn", "swa", "nope"):
            a = lp + "self_attn."
            qkv = w[f"{p}.attn.qkv"]
            qw = cfg.n_head * D * (2 if cfg.gated_attn else 1)
            put(a + "q_proj", qkv[:qw])
            put(a + "k_proj", qkv[qw:qw + cfg.n_kv_head * D])
            put(a + "v_proj", qkv[qw + cfg.n_kv_head * D:])
            if cfg.qk_norm:
                t[a + "q_norm.weight"] = w[f"{p}.attn.q_norm"].cpu().to(dtype)
                t[a + "k_norm.weight"] = w[f"{p}.attn.k_norm"].cpu().to(dtype)
            put(a + "o_proj", w[f"{p}.attn.o"])
        elif kind == "gdn":
            a = lp + "linear_attn."
            nv = cfg.gdn_v_heads
            put(a + "in_proj_qkv", w[f"{p}.gdn.in_qkv"])
            put(a + "in_proj_z", w[f"{p}.gdn.in_z"])
            put(a + "in_proj_b", w[f"{p}.gdn.in_ba"][:nv], False)
            put(a + "in_proj_a", w[f"{p}.gdn.in_ba"][nv:], False)
            t[a + "conv1d.weight"] = w[f"{p}.gdn.conv_w"].cpu().float().unsqueeze(1)
            t[a + "A_log"] = torch.log(-w[f"{p}.gdn.A"].cpu().float())
            t[a + "dt_bias"] = w[f"{p}.gdn.dt_bias"].cpu().float()
            t[a + "norm.weight"] = w[f"{p}.gdn.norm"].cpu().to(dtype)
            put(a + "out_proj", w[f"{p}.gdn.out"])
        elif kind == "mla":
            a = lp + "self_attn."
            inv = lambda x, nh, dn, dr: _interleave_rope(x, nh, dn, dr)
            if cfg.q_lora:
                put(a + "q_a_proj", w[f"{p}.mla.q_a"])
                t[a + "q_a_layernorm.weight"] = w[f"{p}.mla.q_a_norm"].cpu().to(dtype)
                put(a + "q_b_proj", inv(w[f"{p}.mla.q_b"], cfg.n_head, cfg.qk_nope_dim, cfg.qk_rope_dim))
            else:
                put(a + "q_proj", inv(w[f"{p}.mla.q"], cfg.n_head, cfg.qk_nope_dim, cfg.qk_rope_dim))
            put(a + "kv_a_proj_with_mqa", inv(w[f"{p}.mla.kv_a"], 1, cfg.kv_lora, cfg.qk_rope_dim))
            t[a + "kv_a_layernorm.weight"] = w[f"{p}.mla.kv_a_norm"].cpu().to(dtype)
            put(a + "kv_b_proj", w[f"{p}.mla.kv_b"])
            put(a + "o_proj", w[f"{p}.mla.o"])
        if moe_block:
            pre = lp + "mlp."
            put(pre + "gate", w[f"{p}.moe.router"], False)
            if f"{p}.moe.router_bias" in w:
                t[pre + "gate.e_score_correction_bias"] = w[f"{p}.moe.router_bias"].cpu().float()
            F = cfg.expert_ff
            for e in range(cfg.n_expert):
                put(f"{pre}experts.{e}.gate_proj", w[f"{p}.moe.gate_up"][e, :F])
                put(f"{pre}experts.{e}.up_proj", w[f"{p}.moe.gate_up"][e, F:])
                put(f"{pre}experts.{e}.down_proj", w[f"{p}.moe.down"][e])
            if cfg.shared_ff:
                sh = "shared_experts." if cfg.arch == "deepseek_v3" else "shared_expert."
                Fs = cfg.shared_ff
                put(pre + sh + "gate_proj", w[f"{p}.moe.sh_gate_up"][:Fs])
                put(pre + sh + "up_proj", w[f"{p}.moe.sh_gate_up"][Fs:])
                put(pre + sh + "down_proj", w[f"{p}.moe.sh_down"])
                if cfg.shared_gate:
                    put(pre + "shared_expert_gate", w[f"{p}.moe.sh_gate"], False)
        elif cfg.dense_ff:
            F = w[f"{p}.mlp.down"].shape[1]
            put(lp + "mlp.gate_proj", w[f"{p}.mlp.gate_up"][:F])
            put(lp + "mlp.up_proj", w[f"{p}.mlp.gate_up"][F:])
            put(lp + "mlp.down_proj", w[f"{p}.mlp.down"])
    save_file(t, os.path.join(path, "model.safetensors"), {"format": "pt"})
    json.dump(hf_config_dict(cfg, quant), open(os.path.join(path, "config.json"), "w"), indent=1)


def _interleave_rope(wt, n_head, d_nope, d_rope):
    per = d_nope + d_rope
    t = wt.view(n_head, per, -1)
    idx = torch.cat([torch.arange(0, d_rope, 2), torch.arange(1, d_rope, 2)])
    inv = torch.empty_like(idx)
    inv[idx] = torch.arange(d_rope)
    full = torch.cat([torch.arange(d_nope), inv + d_nope])
    # row j of the stored tensor is row full[j] ... invert the permutation used at load time
    out = torch.empty_like(t)
    perm = torch.cat([torch.arange(d_nope), idx + d_nope])
    out[:, perm] = t
    _ = full
    return out.reshape(n_head * per, -1).contiguous()


def hf_config_dict(cfg: ModelConfig, quant: str = "none") -> dict:
    d = {"hidden_size": cfg.hidden, "num_hidden_layers": cfg.n_layer, "num_attention_heads": cfg.n_head,
         "num_key_value_heads": cfg.n_kv_head, "head_dim": cfg.head_dim, "vocab_size": cfg.vocab,
         "rope_theta": cfg.rope_theta, "rms_norm_eps": cfg.rms_eps, "tie_word_embeddings": cfg.tie_embeddings,
         "max_position_embeddings": cfg.max_position, "torch_dtype": "bfloat16"}
    if cfg.arch in ("qwen35", "qwen35moe"):
        d.update(model_type="qwen3_5_moe" if cfg.n_expert else "qwen3_5", mtp_num_hidden_layers=cfg.mtp_layers,
                 layer_types=["linear_attention" if k == "gdn" else "full_attention" for k in cfg.layer_kinds],
                 partial_rotary_factor=cfg.rope_dim / cfg.head_dim, linear_num_key_heads=cfg.gdn_k_heads,
                 linear_num_value_heads=cfg.gdn_v_heads, linear_key_head_dim=cfg.gdn_k_dim,
                 linear_value_head_dim=cfg.gdn_v_dim, linear_conv_kernel_dim=cfg.gdn_conv)
    elif cfg.arch == "deepseek_v3":
        d.update(model_type="deepseek_v3", num_nextn_predict_layers=cfg.mtp_layers,
                 q_lora_rank=cfg.q_lora or None, kv_lora_rank=cfg.kv_lora,
                 qk_nope_head_dim=cfg.qk_nope_dim, qk_rope_head_dim=cfg.qk_rope_dim, v_head_dim=cfg.v_head_dim,
                 intermediate_size=cfg.dense_ff, first_k_dense_replace=cfg.first_dense_layers,
                 n_routed_experts=cfg.n_expert, num_experts_per_tok=cfg.top_k, moe_intermediate_size=cfg.expert_ff,
                 n_shared_experts=(cfg.shared_ff // cfg.expert_ff) if cfg.expert_ff else 0, scoring_func=cfg.router_mode,
                 topk_method="noaux_tc" if cfg.router_bias else "greedy", n_group=cfg.n_group,
                 topk_group=cfg.topk_group, routed_scaling_factor=cfg.route_scale, norm_topk_prob=cfg.norm_topk)
    else:
        d["model_type"] = "qwen3_moe" if cfg.n_expert else ("qwen3" if cfg.qk_norm else "llama")
    if cfg.arch != "deepseek_v3":
        if cfg.n_expert:
            d.update(num_experts=cfg.n_expert, num_experts_per_tok=cfg.top_k, moe_intermediate_size=cfg.expert_ff,
                     norm_topk_prob=cfg.norm_topk, shared_expert_intermediate_size=cfg.shared_ff)
        else:
            d["intermediate_size"] = cfg.dense_ff
    if quant == "fp8_block":
        d["quantization_config"] = {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [128, 128]}
    elif quant == "nvfp4":
        d["quantization_config"] = {"quant_method": "modelopt", "quant_algo": "NVFP4"}
    elif quant == "nvfp4_ct":
        d["quantization_config"] = {"quant_method": "compressed-tensors", "format": "nvfp4-pack-quantized"}
    return d
