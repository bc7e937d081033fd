"""Model hyper-parameters (one dataclass for every supported architecture) and named presets.

The reference keeps these in ``Hparams`` read from GGUF metadata (``src/model/core.rs:170-203``) plus
per-architecture hooks (``src/model/core/arch.rs:82-526``); here every architecture is a configuration of
the same block library, selected by ``layer_kinds`` and the MoE / attention fields.
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class ModelConfig:
    arch: str = "qwen3moe"             # registry key (see models.registry)
    n_layer: int = 4
    hidden: int = 256
    vocab: int = 4096
    rms_eps: float = 1e-6
    norm_offset: float = 0.0           # 1.0 for checkpoints that store (weight - 1)
    tie_embeddings: bool = False
    max_position: int = 131072
    # attention
    n_head: int = 4
    n_kv_head: int = 2
    head_dim: int = 64
    rope_theta: float = 1e6
    rope_dim: Optional[int] = None     # rotary dims per head (None = head_dim); multiple of 64
    rope_scaling: Optional[dict] = None
    mrope_sections: Optional[tuple] = None     # multi-section rotary embedding: frequencies per (temporal, row, column) axis
    mrope_interleaved: bool = True             # axes alternate over the frequencies (Qwen3-VL) or take consecutive sections
    qk_norm: bool = True
    gated_attn: bool = False           # q projection emits [q | gate] per head, out *= sigmoid(gate)
    sliding_window: int = 0            # window of "swa" layers
    attn_softcap: float = 0.0
    logit_softcap: float = 0.0
    logit_scale: float = 1.0           # multiplies the logits before the soft cap (muse-glimmer)
    attn_scale: Optional[float] = None
    # layer pattern: one of "attn", "swa", "nope" (attention without RoPE), "gdn", "mla", "mamba2", "kda" per layer
    layer_kinds: Optional[List[str]] = None
    full_attention_interval: int = 0   # >0: layer il is "gdn" unless (il + 1) % interval == 0
    # gated delta net
    gdn_k_heads: int = 4
    gdn_v_heads: int = 4
    gdn_k_dim: int = 64
    gdn_v_dim: int = 64
    gdn_conv: int = 4
    gdn_tiled_heads: bool = False      # value head h reads key head h % n_k (GGUF order) instead of h // (n_v/n_k)
    gdn_gate_act: str = "silu"         # activation of z in the gated output norm
    # Kimi delta attention ("kda" layers): per-channel decay, q / k / v each behind a short causal convolution
    kda_heads: int = 4
    kda_head_dim: int = 64
    kda_conv: int = 4
    kda_rank: int = 32                 # width of the low-rank gate projections (f_a / f_b, g_a / g_b)
    kda_lower: float = -5.0            # lower bound of the log decay: g = lower * sigmoid(-(f(x) + dt_bias) * A)
    # hyper-connections: the residual is ``hyper_streams`` parallel streams mixed before and after every sublayer
    hyper_streams: int = 1
    hyper_mode: str = "sinkhorn"       # "sinkhorn": per-token pre / post weights and a Sinkhorn-normalised stream mix
                                       # (glm5-next, deepseek41); "gated": a low-rank sigmoid gate per channel mixes
                                       # the normed streams, the block output re-enters every stream with a weight
                                       # of its own, the last mixer is the output norm (qwen4exp)
    hc_rank: int = 16                  # "gated": width of the low-rank gate
    hc_iters: int = 20                 # Sinkhorn rounds of the stream-to-stream mix
    hc_eps: float = 1e-6
    # mamba2 (nemotron-h)
    ssm_state: int = 128
    ssm_heads: int = 8
    ssm_head_dim: int = 64
    ssm_groups: int = 1
    ssm_conv: int = 4
    # MLA
    q_lora: int = 0
    kv_lora: int = 0
    qk_nope_dim: int = 0
    qk_rope_dim: int = 0
    v_head_dim: int = 0
    # feed-forward
    ffn_act: str = "silu"              # silu | gelu_tanh | relu2
    dense_ff: int = 0                  # FFN width of dense layers
    first_dense_layers: int = 0        # leading layers that use the dense FFN in a MoE model
    n_expert: int = 0
    top_k: int = 0
    expert_ff: int = 0
    moe_latent: int = 0                # > 0: the routed experts run at this width, between a down and an up projection
    shared_ff: int = 0                 # width of the shared expert (0 = none)
    shared_gate: bool = False          # sigmoid(x . w) gate on the shared expert
    router_mode: str = "softmax"       # softmax | sigmoid
    router_bias: bool = False          # selection bias (sigmoid routers)
    norm_topk: bool = True
    route_scale: float = 1.0
    n_group: int = 1
    topk_group: int = 1
    # Gemma-4 layer form (``sandwich_norm``): every sublayer between a pre and a post RMS norm, embedding scaled by
    # sqrt(hidden), sliding-window and global layers with head sizes / kv-head counts / rotary bases of their own,
    # values RMS-normed without a weight, unscaled attention, optional: global layers that use their keys as values,
    # trailing layers that read an earlier layer's KV, a per-layer output scale, per-layer token embeddings, and in MoE
    # layers the dense FFN beside the routed experts (router on the normed residual scaled by 1 / sqrt(hidden))
    sandwich_norm: bool = False
    # one sub-layer per block (Nemotron-H as shipped): ``layer_kinds`` then also holds "ffn" and "moe" entries, and a
    # block is x + sublayer(norm(x)) with the mixer OR the feed-forward part, not both
    block_form: bool = False
    embed_scale: float = 1.0
    swa_head_dim: int = 0              # 0 = head_dim
    swa_kv_heads: int = 0              # 0 = n_kv_head
    rope_theta_swa: float = 0.0        # 0 = rope_theta
    rope_freq_factors: Optional[list] = None      # global layers: per-frequency divisors of the rotary frequencies
    v_norm: bool = False
    global_k_as_v: bool = False
    kv_shared_layers: int = 0
    layer_out_scale: bool = False
    ple_dim: int = 0                   # width of the per-layer token embeddings (0 = none)
    # multi-token prediction
    mtp_layers: int = 0
    # weights
    dtype: str = "bf16"                # compute dtype on GPU: bf16; CPU engine uses fp32
    quant: str = "none"                # none | nvfp4 | fp8_block

    def __post_init__(self):
        if self.rope_dim is None:
            self.rope_dim = self.head_dim if not self.qk_rope_dim else self.qk_rope_dim
        if self.layer_kinds is None:
            if self.full_attention_interval > 0:
                self.layer_kinds = ["attn" if (il + 1) % self.full_attention_interval == 0 else "gdn"
                                    for il in range(self.n_layer)]
            elif self.kv_lora > 0:
                self.layer_kinds = ["mla"] * self.n_layer
            else:
                self.layer_kinds = ["attn"] * self.n_layer
        assert len(self.layer_kinds) == self.n_layer

    # ---- derived
    def is_moe_layer(self, il: int) -> bool:
        if self.block_form:
            return il < len(self.layer_kinds) and self.layer_kinds[il] == "moe"
        return self.n_expert > 0 and il >= self.first_dense_layers

    def kv_layers(self) -> List[int]:
        return [i for i, k in enumerate(self.layer_kinds) if k in ("attn", "swa", "nope", "mla")]

    def recurrent_layers(self) -> List[int]:
        return [i for i, k in enumerate(self.layer_kinds) if k in ("gdn", "mamba2", "kda")]

    def kv_dims(self, il: int):
        """(n_kv_heads, k_dim, v_dim) stored per token for layer il."""
        if self.layer_kinds[il] == "mla":
            return 1, self.kv_lora + self.qk_rope_dim, 0
        d, n_kv = self.attn_dims(il)
        return n_kv, d, d

    def attn_dims(self, il: int):
        """(head size, kv heads) of attention layer il: sliding-window layers may have their own."""
        if self.layer_kinds[il] == "swa":
            return self.swa_head_dim or self.head_dim, self.swa_kv_heads or self.n_kv_head
        return self.head_dim, self.n_kv_head

    def owns_kv(self, il: int) -> bool:
        """False for the trailing layers that read another layer's KV cache (``kv_shared_layers``)."""
        return il < self.n_layer - self.kv_shared_layers

    def kv_source(self, il: int) -> int:
        """The layer whose KV cache layer il reads: itself, or the last layer of its kind before the shared ones."""
        if self.owns_kv(il):
            return il
        for j in range(self.n_layer - self.kv_shared_layers - 1, -1, -1):
            if self.layer_kinds[j] == self.layer_kinds[il]:
                return j
        raise ValueError(f"layer {il} shares a KV cache but no earlier layer of its kind owns one")

    def has_v_proj(self, il: int) -> bool:
        return not (self.global_k_as_v and self.layer_kinds[il] != "swa")

    def gdn_conv_channels(self) -> int:
        return 2 * self.gdn_k_heads * self.gdn_k_dim + self.gdn_v_heads * self.gdn_v_dim

    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self))

    @classmethod
    def from_dict(cls, d: dict) -> "ModelConfig":
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in names})

    def param_count(self) -> int:
        from .models.weights import weight_shapes
        n = 0
        for shp in weight_shapes(self).values():
            m = 1
            for s in shp:
                m *= s
            n += m
        return n


# --------------------------------------------------------------------------------------------------
# presets
# --------------------------------------------------------------------------------------------------
def tiny_glm_next() -> "ModelConfig":
    """Shape of the glm5-next family in miniature: Kimi-delta-attention layers with a latent-attention layer every
    third, hyper-connections (4 streams) around every sublayer, sigmoid-routed MoE with a shared expert after one
    dense layer. The latent-attention layers attend densely (no sparse key selection)."""
    return ModelConfig(arch="glm5_next", n_layer=3, hidden=128, vocab=512, n_head=4, n_kv_head=4, head_dim=96,
                       layer_kinds=["kda", "kda", "mla"], kda_heads=4, kda_head_dim=32, kda_rank=16,
                       q_lora=48, kv_lora=64, qk_nope_dim=32, qk_rope_dim=64, v_head_dim=32, qk_norm=False,
                       hyper_streams=4, hc_iters=8, dense_ff=192, first_dense_layers=1, n_expert=8, top_k=2,
                       expert_ff=64, shared_ff=64, router_mode="sigmoid", router_bias=True, route_scale=2.0)


def tiny_qwen4exp() -> "ModelConfig":
    """Shape of the qwen4exp family in miniature: the hybrid Gated-DeltaNet / gated-attention MoE stack with a
    sigmoid DeltaNet output gate, multi-section rotary positions and gated hyper-connections (4 streams) in place of
    the residual stream and the pre-norms. Attention is dense (its sparse key selection equals dense attention up to
    the selection budget); the n-gram embedding layer is not modelled."""
    c = tiny_hybrid_moe()
    c.arch = "qwen4exp"
    c.hyper_streams, c.hyper_mode, c.hc_rank = 4, "gated", 8
    c.gdn_gate_act = "sigmoid"
    if c.rope_dim == 64:
        c.mrope_sections = (11, 11, 10)
    return c


def tiny_hybrid_moe() -> ModelConfig:
    """4-layer hybrid: 3 Gated DeltaNet layers + 1 gated GQA layer, 8 experts top-2 + shared expert."""
    return ModelConfig(arch="qwen35moe", n_layer=4, hidden=256, vocab=4096, n_head=4, n_kv_head=2, head_dim=64,
                       rope_theta=1e6, full_attention_interval=4, gated_attn=True, gdn_k_heads=4, gdn_v_heads=4,
                       gdn_k_dim=64, gdn_v_dim=64, gdn_conv=4, n_expert=8, top_k=2, expert_ff=512, shared_ff=512,
                       shared_gate=True)


def tiny_gqa_moe() -> ModelConfig:
    return ModelConfig(arch="qwen3moe", n_layer=2, hidden=256, vocab=1024, n_head=4, n_kv_head=2, head_dim=64,
                       n_expert=8, top_k=2, expert_ff=128)


def tiny_dense() -> ModelConfig:
    return ModelConfig(arch="qwen3", n_layer=2, hidden=256, vocab=1024, n_head=4, n_kv_head=2, head_dim=64,
                       dense_ff=512)


def tiny_mla_moe() -> ModelConfig:
    return ModelConfig(arch="deepseek_v3", n_layer=3, hidden=256, vocab=1024, n_head=4, n_kv_head=4, head_dim=96,
                       q_lora=96, kv_lora=64, qk_nope_dim=32, qk_rope_dim=64, v_head_dim=32, qk_norm=False,
                       dense_ff=384, first_dense_layers=1, n_expert=8, top_k=2, expert_ff=128, shared_ff=128,
                       router_mode="sigmoid", router_bias=True, n_group=4, topk_group=2, route_scale=2.5,
                       mtp_layers=1)


def qwen3_30b_a3b() -> ModelConfig:
    """30B-A3B-shape MoE: 48 layers, 128 experts top-8, no shared expert."""
    return ModelConfig(arch="qwen3moe", n_layer=48, hidden=2048, vocab=151936, n_head=32, n_kv_head=4, head_dim=128,
                       rope_theta=1e6, n_expert=128, top_k=8, expert_ff=768)


def qwen35_80b_a3b() -> ModelConfig:
    """80B-A3B-shape hybrid MoE: 3:1 Gated DeltaNet to gated attention, 512 experts top-10 + shared."""
    return ModelConfig(arch="qwen35moe", n_layer=48, hidden=2048, vocab=151936, n_head=16, n_kv_head=2, head_dim=256,
                       rope_dim=64, rope_theta=1e7, full_attention_interval=4, gated_attn=True, gdn_k_heads=16,
                       gdn_v_heads=32, gdn_k_dim=128, gdn_v_dim=128, gdn_conv=4, n_expert=512, top_k=10,
                       expert_ff=512, shared_ff=512, shared_gate=True, norm_offset=0.0, quant="nvfp4")


def deepseek_671b() -> ModelConfig:
    """671B-shape MLA MoE: 61 layers, 256 routed experts top-8 (8 groups, top-4), 1 shared expert, 1 MTP head."""
    return ModelConfig(arch="deepseek_v3", n_layer=61, hidden=7168, vocab=129280, n_head=128, n_kv_head=128,
                       head_dim=192, q_lora=1536, kv_lora=512, qk_nope_dim=128, qk_rope_dim=64, v_head_dim=128,
                       qk_norm=False, rope_theta=1e4, dense_ff=18432, first_dense_layers=3, n_expert=256, top_k=8,
                       expert_ff=2048, shared_ff=2048, router_mode="sigmoid", router_bias=True, n_group=8,
                       topk_group=4, route_scale=2.5, mtp_layers=1, quant="fp8_block")


def dense_27b() -> ModelConfig:
    return ModelConfig(arch="qwen3", n_layer=64, hidden=5120, vocab=151936, n_head=40, n_kv_head=8, head_dim=128,
                       rope_theta=1e6, dense_ff=17408)


def tiny_muse() -> ModelConfig:
    """muse-glimmer shape: dense, sliding-window RoPE layers with every third layer global without RoPE, QK norm,
    sigmoid output gate, logit scale + soft cap (``src/model/muse.rs:1-25`` in the reference)."""
    return ModelConfig(arch="muse-glimmer", n_layer=6, hidden=256, vocab=4096, n_head=4, n_kv_head=2, head_dim=64,
                       layer_kinds=["swa", "swa", "nope", "swa", "swa", "nope"], sliding_window=32, gated_attn=True,
                       dense_ff=512, logit_scale=0.5, logit_softcap=30.0)


def tiny_gemma() -> ModelConfig:
    """Gemma-style: alternating sliding-window / global attention, GELU-gated FFN, (weight - 1) norm storage,
    tied embeddings, logit soft cap 30 (``src/model/gemma4.rs:1-30``; per-layer head sizes and shared-KV layers of
    Gemma 4 are not modelled)."""
    return ModelConfig(arch="gemma4", n_layer=4, hidden=256, vocab=4096, n_head=4, n_kv_head=2, head_dim=64,
                       layer_kinds=["swa", "attn", "swa", "attn"], sliding_window=48, ffn_act="gelu_tanh",
                       dense_ff=512, norm_offset=1.0, tie_embeddings=True, logit_softcap=30.0)


def tiny_nemotron_h() -> ModelConfig:
    """Nemotron-H style hybrid: Mamba-2 layers with a few attention layers without RoPE, squared-ReLU FFN
    (``src/model/nemotron_h.rs:1-20``; latent MoE and per-layer expert counts are not modelled)."""
    return ModelConfig(arch="nemotron_h", n_layer=4, hidden=256, vocab=4096, n_head=4, n_kv_head=2, head_dim=64,
                       layer_kinds=["mamba2", "mamba2", "nope", "mamba2"], qk_norm=False, ffn_act="relu2",
                       dense_ff=512, ssm_state=32, ssm_heads=8, ssm_head_dim=32, ssm_groups=1, ssm_conv=4)


def tiny_nemotron_h_moe() -> ModelConfig:
    """The Nemotron-H hybrid with its latent MoE (``src/model/nemotron_h.rs:538-608``): the router reads the normed
    input, the routed squared-ReLU experts run at ``moe_latent`` between ``lat_down`` and ``lat_up``, the shared
    expert at full width."""
    c = tiny_nemotron_h()
    c.dense_ff, c.first_dense_layers = 512, 1
    c.n_expert, c.top_k, c.expert_ff, c.shared_ff, c.moe_latent = 8, 2, 128, 128, 128
    c.router_mode, c.router_bias, c.norm_topk, c.route_scale = "sigmoid", True, True, 2.5
    return c


def tiny_nemotron_h_blocks() -> ModelConfig:
    """Nemotron-H the way its checkpoints lay it out: one sub-layer per block (``block_form``), here Mamba-2 with two
    norm groups, a dense squared-ReLU FFN, attention without rotary embedding, and the latent MoE."""
    c = tiny_nemotron_h_moe()
    c.block_form, c.first_dense_layers, c.ssm_groups = True, 0, 2
    c.layer_kinds = ["mamba2", "ffn", "nope", "moe", "mamba2", "moe"]
    c.n_layer = len(c.layer_kinds)
    return c


def tiny_gemma4() -> ModelConfig:
    """Gemma 4 in miniature (``src/model/gemma4.rs:1-30``): sandwich norms, scaled embedding, sliding-window layers
    with 64-wide heads and 2 kv heads next to global layers with 128-wide heads, 1 kv head, keys used as values and
    rotary frequency factors, value norm, unscaled attention, the last two layers reading earlier layers' KV, a
    per-layer output scale, per-layer token embeddings, and MoE layers whose dense GELU FFN runs beside 8 routed GELU
    experts."""
    return ModelConfig(arch="gemma4", n_layer=6, hidden=256, vocab=4096, n_head=4, n_kv_head=1, head_dim=128,
                       layer_kinds=["swa", "swa", "attn", "swa", "swa", "attn"], sliding_window=48, rope_dim=128,
                       rope_theta=1e6, rope_freq_factors=[1.0] * 48 + [8.0] * 16, swa_head_dim=64, swa_kv_heads=2,
                       rope_theta_swa=1e4, ffn_act="gelu_tanh", dense_ff=384, norm_offset=0.0, tie_embeddings=True,
                       logit_softcap=30.0, attn_scale=1.0, sandwich_norm=True, embed_scale=16.0, v_norm=True,
                       global_k_as_v=True, kv_shared_layers=2, layer_out_scale=True, ple_dim=32, first_dense_layers=1,
                       n_expert=8, top_k=2, expert_ff=128, router_mode="softmax", norm_topk=True)


PRESETS = {
    "tiny-muse": tiny_muse,
    "tiny-gemma4": tiny_gemma4,
    "tiny-nemotron-h-moe": tiny_nemotron_h_moe,
    "tiny-nemotron-h-blocks": tiny_nemotron_h_blocks,
    "tiny-gemma": tiny_gemma,
    "tiny-nemotron-h": tiny_nemotron_h,
    "tiny-hybrid-moe": tiny_hybrid_moe,
    "tiny-glm-next": tiny_glm_next,
    "tiny-qwen4exp": tiny_qwen4exp,
    "tiny-gqa-moe": tiny_gqa_moe,
    "tiny-dense": tiny_dense,
    "tiny-mla-moe": tiny_mla_moe,
    "qwen3-30b-a3b": qwen3_30b_a3b,
    "qwen35-80b-a3b": qwen35_80b_a3b,
    "deepseek-671b": deepseek_671b,
    "dense-27b": dense_27b,
}
