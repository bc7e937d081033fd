"""Canonical weight names, shapes, random initialisation and tensor-parallel / expert-parallel sharding.

Names are architecture-neutral (``l{i}.attn.qkv`` ...); the GGUF and safetensors loaders map their own
names onto these (``loaders/gguf_map.py``, ``loaders/hf_map.py``). Projections that one kernel consumes
together are stored fused: q/k/v, gate/up, and the per-expert stacks, like the reference's stacked 3-D
expert tensors (``src/hf/qwen35.rs:6-20``).

Sharding follows the Megatron rule the reference uses (``src/model/core/tp.rs:110``): q/k/v/gate/up by
output rows (whole heads), o/down by input columns, experts whole under EP, everything else mirrored.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..config import ModelConfig


def layer_weight_shapes(cfg: ModelConfig, il: int, prefix: Optional[str] = None, kind: Optional[str] = None,
                        moe: Optional[bool] = None) -> Dict[str, Tuple[int, ...]]:
    p = prefix if prefix is not None else f"l{il}"
    kind = kind or cfg.layer_kinds[il]
    moe = cfg.is_moe_layer(il) if moe is None else moe
    H = cfg.hidden
    if cfg.block_form and prefix is None:
        # one sub-layer per block: its input norm plus either the mixer's or the feed-forward part's tensors
        if kind in ("ffn", "moe"):
            return _ffn_shapes(cfg, p, kind == "moe", {f"{p}.attn_norm": (H,)})
        full = layer_weight_shapes(cfg, il, prefix=p, kind=kind, moe=False)
        return {k: v for k, v in full.items() if not (k.startswith(f"{p}.mlp.") or k == f"{p}.ffn_norm")}
    s: Dict[str, Tuple[int, ...]] = {f"{p}.attn_norm": (H,), f"{p}.ffn_norm": (H,)}
    if cfg.sandwich_norm and kind in ("attn", "swa") and prefix is None:
        return gemma_layer_shapes(cfg, il, s)
    if kind in ("attn", "swa", "nope"):
        D = cfg.head_dim
        qw = cfg.n_head * D * (2 if cfg.gated_attn else 1)
        s[f"{p}.attn.qkv"] = (qw + 2 * cfg.n_kv_head * D, H)
        if cfg.qk_norm:
            s[f"{p}.attn.q_norm"] = (D,)
            s[f"{p}.attn.k_norm"] = (D,)
        s[f"{p}.attn.o"] = (H, cfg.n_head * D)
    elif kind == "gdn":
        C = cfg.gdn_conv_channels()
        nv, dv = cfg.gdn_v_heads, cfg.gdn_v_dim
        s[f"{p}.gdn.in_qkv"] = (C, H)
        s[f"{p}.gdn.in_z"] = (nv * dv, H)
        s[f"{p}.gdn.in_ba"] = (2 * nv, H)
        s[f"{p}.gdn.conv_w"] = (C, cfg.gdn_conv)
        s[f"{p}.gdn.A"] = (nv,)
        s[f"{p}.gdn.dt_bias"] = (nv,)
        s[f"{p}.gdn.norm"] = (dv,)
        s[f"{p}.gdn.out"] = (H, nv * dv)
    elif kind == "mla":
        nh = cfg.n_head
        if cfg.q_lora > 0:
            s[f"{p}.mla.q_a"] = (cfg.q_lora, H)
            s[f"{p}.mla.q_a_norm"] = (cfg.q_lora,)
            s[f"{p}.mla.q_b"] = (nh * (cfg.qk_nope_dim + cfg.qk_rope_dim), cfg.q_lora)
        else:
            s[f"{p}.mla.q"] = (nh * (cfg.qk_nope_dim + cfg.qk_rope_dim), H)
        s[f"{p}.mla.kv_a"] = (cfg.kv_lora + cfg.qk_rope_dim, H)
        s[f"{p}.mla.kv_a_norm"] = (cfg.kv_lora,)
        s[f"{p}.mla.kv_b"] = (nh * (cfg.qk_nope_dim + cfg.v_head_dim), cfg.kv_lora)
        s[f"{p}.mla.o"] = (H, nh * cfg.v_head_dim)
    elif kind == "kda":
        c, r = cfg.kda_heads * cfg.kda_head_dim, cfg.kda_rank
        s[f"{p}.kda.qkv"] = (3 * c, H)                  # q | k | v, each heads x head_dim
        s[f"{p}.kda.conv_w"] = (3 * c, cfg.kda_conv)
        s[f"{p}.kda.f_a"] = (r, H)                      # decay gate, low rank: f_b (f_a x)
        s[f"{p}.kda.f_b"] = (c, r)
        s[f"{p}.kda.dt_bias"] = (c,)
        s[f"{p}.kda.A"] = (cfg.kda_heads,)
        s[f"{p}.kda.beta"] = (cfg.kda_heads, H)
        s[f"{p}.kda.g_a"] = (r, H)                      # output gate, low rank: g_b (g_a x)
        s[f"{p}.kda.g_b"] = (c, r)
        s[f"{p}.kda.norm"] = (cfg.kda_head_dim,)
        s[f"{p}.kda.out"] = (H, c)
    elif kind == "mamba2":
        di = cfg.ssm_heads * cfg.ssm_head_dim
        conv_c = di + 2 * cfg.ssm_groups * cfg.ssm_state
        s[f"{p}.ssm.in"] = (2 * di + 2 * cfg.ssm_groups * cfg.ssm_state + cfg.ssm_heads, H)
        s[f"{p}.ssm.conv_w"] = (conv_c, cfg.ssm_conv)
        s[f"{p}.ssm.conv_b"] = (conv_c,)
        s[f"{p}.ssm.A"] = (cfg.ssm_heads,)
        s[f"{p}.ssm.D"] = (cfg.ssm_heads,)
        s[f"{p}.ssm.dt_bias"] = (cfg.ssm_heads,)
        s[f"{p}.ssm.norm"] = (di,)
        s[f"{p}.ssm.out"] = (H, di)
    else:
        raise ValueError(f"unknown layer kind {kind}")
    if cfg.hyper_streams > 1:
        hc = cfg.hyper_streams
        for which in ("hca", "hcf"):                    # the mixers in front of the attention and the FFN sublayer
            if cfg.hyper_mode == "gated":
                s.update(gated_mixer_shapes(cfg, f"{p}.{which}", inject=True))
                continue
            s[f"{p}.{which}.hc_f"] = ((2 + hc) * hc, hc * H)
            s[f"{p}.{which}.hc_scale"] = (3,)
            s[f"{p}.{which}.hc_base"] = ((2 + hc) * hc,)
        if cfg.hyper_mode == "gated":                   # the mixers take the place of the pre-norms
            s.pop(f"{p}.attn_norm", None)
            s.pop(f"{p}.ffn_norm", None)
    return _ffn_shapes(cfg, p, moe, s)


def _ffn_shapes(cfg: ModelConfig, p: str, moe: bool, s: Dict[str, Tuple[int, ...]]) -> Dict[str, Tuple[int, ...]]:
    """The feed-forward part of a layer: routed experts (router, latent projections, shared expert) or the dense FFN."""
    H = cfg.hidden
    if moe:
        E, F = cfg.n_expert, cfg.expert_ff
        s[f"{p}.moe.router"] = (E, H)
        if cfg.router_bias:
            s[f"{p}.moe.router_bias"] = (E,)
        gu = 2 * F if cfg.ffn_act != "relu2" else F
        W = cfg.moe_latent or H                         # width the routed experts run at
        if cfg.moe_latent:
            s[f"{p}.moe.lat_down"] = (W, H)
            s[f"{p}.moe.lat_up"] = (H, W)
        s[f"{p}.moe.gate_up"] = (E, gu, W)
        s[f"{p}.moe.down"] = (E, W, F)
        if cfg.shared_ff > 0:
            s[f"{p}.moe.sh_gate_up"] = (2 * cfg.shared_ff if cfg.ffn_act != "relu2" else cfg.shared_ff, H)
            s[f"{p}.moe.sh_down"] = (H, cfg.shared_ff)
            if cfg.shared_gate:
                s[f"{p}.moe.sh_gate"] = (1, H)
    elif cfg.dense_ff > 0:
        F = cfg.dense_ff
        s[f"{p}.mlp.gate_up"] = (2 * F if cfg.ffn_act != "relu2" else F, H)
        s[f"{p}.mlp.down"] = (H, F)
    return s


def gemma_layer_shapes(cfg: ModelConfig, il: int, s: Dict[str, Tuple[int, ...]]) -> Dict[str, Tuple[int, ...]]:
    """Gemma-4 layer: q (+ k (+ v)) rows of this layer's head size, post norms, optional routed experts beside the
    dense FFN, output scale, per-layer embedding gate / projection."""
    p, H = f"l{il}", cfg.hidden
    D, n_kv = cfg.attn_dims(il)
    rows = cfg.n_head * D
    if cfg.owns_kv(il):
        rows += n_kv * D * (2 if cfg.has_v_proj(il) else 1)
        s[f"{p}.attn.k_norm"] = (D,)
    s[f"{p}.attn.qkv"] = (rows, H)
    s[f"{p}.attn.q_norm"] = (D,)
    s[f"{p}.attn.o"] = (H, cfg.n_head * D)
    s[f"{p}.attn_post_norm"] = (H,)
    s[f"{p}.ffn_post_norm"] = (H,)
    F = cfg.dense_ff
    s[f"{p}.mlp.gate_up"] = (2 * F, H)
    s[f"{p}.mlp.down"] = (H, F)
    if cfg.is_moe_layer(il):
        E, Fe = cfg.n_expert, cfg.expert_ff
        s[f"{p}.ffn_post1_norm"] = (H,)
        s[f"{p}.ffn_pre2_norm"] = (H,)
        s[f"{p}.ffn_post2_norm"] = (H,)
        s[f"{p}.moe.router"] = (E, H)
        s[f"{p}.moe.router_scale"] = (H,)
        s[f"{p}.moe.gate_up"] = (E, 2 * Fe, H)
        s[f"{p}.moe.down"] = (E, H, Fe)
    if cfg.layer_out_scale:
        s[f"{p}.out_scale"] = (1,)
    if cfg.ple_dim:
        s[f"{p}.ple.inp_gate"] = (cfg.ple_dim, H)
        s[f"{p}.ple.proj"] = (H, cfg.ple_dim)
        s[f"{p}.ple.post_norm"] = (H,)
    return s


def gated_mixer_shapes(cfg: ModelConfig, name: str, inject: bool) -> Dict[str, Tuple[int, ...]]:
    hc, H, r = cfg.hyper_streams, cfg.hidden, cfg.hc_rank
    s = {f"{name}.hcg_norm": (hc, H), f"{name}.hcg_down": (r, hc * H), f"{name}.hcg_up": (hc * H, r)}
    if inject:
        s[f"{name}.hcg_inject"] = (hc, hc * H)
    return s


def weight_shapes(cfg: ModelConfig) -> Dict[str, Tuple[int, ...]]:
    s: Dict[str, Tuple[int, ...]] = {"tok_embd": (cfg.vocab, cfg.hidden), "output_norm": (cfg.hidden,)}
    if cfg.sandwich_norm and cfg.ple_dim:
        s["ple_embd"] = (cfg.vocab, cfg.ple_dim * cfg.n_layer)
        s["ple_model_proj"] = (cfg.ple_dim * cfg.n_layer, cfg.hidden)
        s["ple_proj_norm"] = (cfg.ple_dim,)
    if cfg.hyper_streams > 1 and cfg.hyper_mode == "gated":
        s.pop("output_norm")                            # the last mixer is the output norm
        s.update(gated_mixer_shapes(cfg, "out_hc", inject=False))
    if not cfg.tie_embeddings:
        s["output"] = (cfg.vocab, cfg.hidden)
    for il in range(cfg.n_layer):
        s.update(layer_weight_shapes(cfg, il))
    for j in range(cfg.mtp_layers):
        p = f"mtp{j}"
        s[f"{p}.eh_proj"] = (cfg.hidden, 2 * cfg.hidden)
        s[f"{p}.enorm"] = (cfg.hidden,)
        s[f"{p}.hnorm"] = (cfg.hidden,)
        s[f"{p}.shared_head_norm"] = (cfg.hidden,)
        kind = "mla" if cfg.kv_lora > 0 else "attn"
        s.update(layer_weight_shapes(cfg, cfg.n_layer + j, prefix=f"{p}.l", kind=kind, moe=cfg.n_expert > 0))
    return s


FP32_SUFFIXES = ("_norm", ".norm", "norm", ".A", ".D", ".dt_bias", ".conv_w", ".conv_b", ".router_bias", ".q_norm",
                 ".k_norm", ".sh_gate")


def is_fp32_weight(name: str) -> bool:
    """Norm weights, recurrence constants and conv taps stay float32 on every back-end."""
    leaf = name.rsplit(".", 1)[-1]
    return leaf.endswith("norm") or leaf in ("A", "D", "dt_bias", "conv_w", "conv_b", "router_bias", "hc_f", "hc_scale",
                                             "hc_base", "hcg_norm", "hcg_down", "hcg_up", "hcg_inject", "router_scale",
                                             "out_scale")


def layer_of(name: str) -> Optional[int]:
    """Layer index of a canonical weight name (``l12.attn.qkv`` -> 12), None for embeddings / head / MTP."""
    if name.startswith("l") and "." in name and name[1:name.index(".")].isdigit():
        return int(name[1:name.index(".")])
    return None


def random_weights(cfg: ModelConfig, device="cpu", dtype=torch.float32, seed: int = 0, std: float = 0.02,
                   shard: Optional["Shard"] = None, keep=None, post=None) -> Dict[str, torch.Tensor]:
    """N(0, std) matrices; norm weights 1, A in (-1, -0.1), dt_bias small. With ``shard`` only this rank's
    slices are created (device-side generation for models too large for the host). ``keep(name)`` drops
    tensors a pipeline stage does not own; the kept ones equal those of the full model. ``post(name, weights)``
    runs after every tensor and may replace entries of the dictionary (a model whose bf16 form does not fit the
    device is quantised layer by layer while it is generated)."""
    device = torch.device(device)
    out: Dict[str, torch.Tensor] = {}
    g = torch.Generator(device="cpu").manual_seed(seed)
    names = weight_shapes(cfg)
    for idx, (name, shp) in enumerate(names.items()):
        leaf = name.rsplit(".", 1)[-1]
        wd = torch.float32 if is_fp32_weight(name) else dtype
        if shard is not None:
            shp = shard.local_shape(name, shp)
        dropped = keep is not None and not keep(name)
        if dropped and (leaf.endswith("norm") or leaf == "D" or (device.type == "cuda" and wd == torch.bfloat16)):
            continue                      # nothing drawn from the host generator for these
        if leaf.endswith("norm"):
            t = torch.ones(shp, dtype=torch.float32, device=device) - cfg.norm_offset
        elif leaf == "A":
            t = -(torch.rand(shp, generator=g) * 0.9 + 0.1).to(device)
        elif leaf == "D":
            t = torch.ones(shp, dtype=torch.float32, device=device)
        elif leaf in ("dt_bias", "conv_b", "router_bias"):
            t = (torch.randn(shp, generator=g) * 0.1).to(device)
        elif leaf in ("hc_scale", "router_scale", "out_scale"):
            t = torch.ones(shp, dtype=torch.float32, device=device) * (0.9 if leaf == "out_scale" else 1.0)
        elif leaf == "hc_base":
            t = (torch.randn(shp, generator=g) * 0.5).to(device)
        elif leaf in ("hc_f", "hcg_down", "hcg_up", "hcg_inject"):
            t = (torch.randn(shp, generator=g) * 0.05).to(device)
        elif leaf == "conv_w":
            t = (torch.randn(shp, generator=g) * 0.3).to(device)
        elif device.type == "cuda" and wd == torch.bfloat16:
            from ..ops.sm100 import ext
            t = torch.empty(shp, dtype=torch.bfloat16, device=device)
            ext().randn_bf16(t, std, seed * 1000003 + idx)
        else:
            t = (torch.randn(shp, generator=g) * std).to(device=device, dtype=wd)
        if not dropped:                   # dropped host-generated tensors still advanced the generator
            out[name] = t.to(wd)
            if post is not None:
                del t
                post(name, out)
    return out


class Shard:
    """Tensor-parallel (attention / dense FFN / shared expert) and expert-parallel slicing of weights."""

    def __init__(self, cfg: ModelConfig, rank: int, world: int, expert_parallel: bool = False,
                 dp_attention: bool = False, shared_whole: bool = False):
        self.cfg, self.rank, self.world, self.ep = cfg, rank, world, expert_parallel or dp_attention
        # the shared expert is not sliced: every rank gets it whole, so that one rank per layer can run it as one
        # more slot of its grouped expert GEMMs (models.decoder.place_shared_expert) and the others drop it
        self.shared_whole = shared_whole
        self.dp_attention = dp_attention     # only the routed experts are split; everything else is whole
        if dp_attention:
            self.kv_rep = 1
            return
        if world > 1 and ("kda" in cfg.layer_kinds or cfg.hyper_streams > 1 or cfg.sandwich_norm or cfg.block_form):
            raise NotImplementedError("Kimi-delta-attention layers, hyper-connections and the Gemma-4 layer form run "
                                      "on one rank (their weights have no tensor-parallel split here)")
        assert cfg.n_head % world == 0, "query heads must divide by the TP degree"
        self.kv_rep = 1
        if cfg.n_kv_head % world != 0:
            assert world % cfg.n_kv_head == 0, "kv heads must divide, or be divided by, the TP degree"
            self.kv_rep = world // cfg.n_kv_head

    # expert range of this rank under EP
    def expert_range(self):
        E = self.cfg.n_expert
        if not self.ep:
            return 0, E
        per = E // self.world
        return self.rank * per, (self.rank + 1) * per

    def _rows(self, n):  # contiguous row block of this rank
        per = n // self.world
        return slice(self.rank * per, (self.rank + 1) * per)

    def plan(self, name: str, shape):
        """Returns a list of (dim, index) selections describing this rank's slice, or None if mirrored."""
        cfg, w, r = self.cfg, self.world, self.rank
        leaf = name.split(".", 1)[1] if "." in name else name
        leaf = leaf.replace("l.", "", 1) if name.startswith("mtp") and leaf.startswith("l.") else leaf
        if w == 1:
            return None
        if self.dp_attention and leaf not in ("moe.gate_up", "moe.down"):
            return None
        if leaf == "attn.qkv":
            D = cfg.head_dim
            qh = D * (2 if cfg.gated_attn else 1)
            nq, nkv = cfg.n_head, cfg.n_kv_head
            q_rows = torch.arange(nq * qh).view(nq, qh)[self._rows(nq)].reshape(-1)
            if self.kv_rep == 1:
                kvh = torch.arange(nkv)[self._rows(nkv)]
            else:
                kvh = torch.tensor([r // self.kv_rep])
            k_rows = (nq * qh + (kvh[:, None] * D + torch.arange(D)[None])).reshape(-1)
            v_rows = k_rows + nkv * D
            return [(0, torch.cat([q_rows, k_rows, v_rows]))]
        if leaf == "attn.o":
            per = shape[1] // w
            return [(1, torch.arange(r * per, (r + 1) * per))]
        if self.shared_whole and leaf in ("moe.sh_gate_up", "moe.sh_down"):
            return None
        if leaf in ("mlp.gate_up", "moe.sh_gate_up"):
            F = shape[0] // 2 if cfg.ffn_act != "relu2" else shape[0]
            per = F // w
            idx = torch.arange(r * per, (r + 1) * per)
            return [(0, torch.cat([idx, idx + F]) if cfg.ffn_act != "relu2" else idx)]
        if leaf in ("mlp.down", "moe.sh_down"):
            per = shape[1] // w
            return [(1, torch.arange(r * per, (r + 1) * per))]
        if leaf in ("moe.gate_up", "moe.down"):
            if self.ep:
                lo, hi = self.expert_range()
                return [(0, torch.arange(lo, hi))]
            if leaf == "moe.gate_up":
                F = shape[1] // 2 if cfg.ffn_act != "relu2" else shape[1]
                per = F // w
                idx = torch.arange(r * per, (r + 1) * per)
                return [(1, torch.cat([idx, idx + F]) if cfg.ffn_act != "relu2" else idx)]
            per = shape[2] // w
            return [(2, torch.arange(r * per, (r + 1) * per))]
        if leaf in ("mla.q_b", "mla.q", "mla.kv_b"):
            nh = cfg.n_head
            per_head = shape[0] // nh
            rows = torch.arange(shape[0]).view(nh, per_head)[self._rows(nh)].reshape(-1)
            return [(0, rows)]
        if leaf == "mla.o":
            per = shape[1] // w
            return [(1, torch.arange(r * per, (r + 1) * per))]
        if leaf == "gdn.in_qkv":
            nk, nv, dk, dv = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_k_dim, cfg.gdn_v_dim
            q = torch.arange(nk * dk).view(nk, dk)[self._rows(nk)].reshape(-1)
            k = q + nk * dk
            v = 2 * nk * dk + torch.arange(nv * dv).view(nv, dv)[self._rows(nv)].reshape(-1)
            return [(0, torch.cat([q, k, v]))]
        if leaf == "gdn.conv_w":
            nk, nv, dk, dv = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_k_dim, cfg.gdn_v_dim
            q = torch.arange(nk * dk).view(nk, dk)[self._rows(nk)].reshape(-1)
            k = q + nk * dk
            v = 2 * nk * dk + torch.arange(nv * dv).view(nv, dv)[self._rows(nv)].reshape(-1)
            return [(0, torch.cat([q, k, v]))]
        if leaf == "gdn.in_z":
            nv, dv = cfg.gdn_v_heads, cfg.gdn_v_dim
            return [(0, torch.arange(nv * dv).view(nv, dv)[self._rows(nv)].reshape(-1))]
        if leaf == "gdn.in_ba":
            nv = cfg.gdn_v_heads
            h = torch.arange(nv)[self._rows(nv)]
            return [(0, torch.cat([h, h + nv]))]
        if leaf in ("gdn.A", "gdn.dt_bias"):
            return [(0, torch.arange(cfg.gdn_v_heads)[self._rows(cfg.gdn_v_heads)])]
        if leaf == "gdn.out":
            nv, dv = cfg.gdn_v_heads, cfg.gdn_v_dim
            return [(1, torch.arange(nv * dv).view(nv, dv)[self._rows(nv)].reshape(-1))]
        return None

    def local_shape(self, name, shape):
        p = self.plan(name, shape)
        if p is None:
            return tuple(shape)
        shp = list(shape)
        for dim, idx in p:
            shp[dim] = int(idx.numel())
        return tuple(shp)

    def slice(self, name: str, t: torch.Tensor) -> torch.Tensor:
        p = self.plan(name, tuple(t.shape))
        if p is None:
            return t
        for dim, idx in p:
            t = t.index_select(dim, idx.to(t.device))
        return t.contiguous()

    def shard_all(self, weights: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        return {k: self.slice(k, v) for k, v in weights.items()}
