"""Config-driven decoder: every supported architecture is a stack of the blocks below.

One forward serves prefill chunks, decode steps and speculative verify steps: the step is a flat list
of tokens (``StepBatch``) grouped into sequences by ``cu_q``; attention reads the paged KV cache through
block tables, recurrent layers read and advance per-sequence state slots. Sequence lengths, block tables
and positions are tensors (data), so a step's kernel sequence depends only on the batch shape: the
property the reference gets from paged attention (``src/model/core/paged.rs:10-13``) and that lets the
GPU engine replay decode steps as CUDA graphs.

Blocks (reference structure in parentheses):
  attn / swa  GQA attention, per-head QK RMS-norm, RoPE, optional sigmoid output gate
              (``src/model/core.rs:3996-4092``)
  gdn         Gated DeltaNet: in-proj -> causal conv1d + SiLU -> L2-normed q,k -> gated delta rule ->
              gated RMS norm -> out-proj (``src/model/core.rs:3484-3984``)
  mla         Multi-head latent attention over a cached [latent | rope-key] row per token
  mamba2      Mamba-2 selective state space layer (``src/model/nemotron_h.rs``)
  moe         router -> top-k -> routed experts (+ shared expert, + sigmoid shared gate)
              (``src/model/core.rs:4496-4640``); dense SwiGLU / GELU / ReLU^2 FFN
  mtp         next-token-prediction head: eh_proj([norm(embed) ; norm(hidden)]) -> one block -> shared
              head norm -> LM head (``src/model/qwen35/mtp.rs:1-14``)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from .. import ops
from ..config import ModelConfig
from ..parallel.context import ParallelCtx, PendingLinear


@dataclass
class StepBatch:
    token_ids: torch.Tensor          # [T] int32
    positions: torch.Tensor          # [T] int32
    cu_q: torch.Tensor               # [n_seqs + 1] int32
    ctx_lens: torch.Tensor           # [n_seqs] int32: cached tokens + this step's tokens
    block_table: torch.Tensor        # [n_seqs, width] int32
    slots: torch.Tensor              # [T] int64 flat KV cell of each token (block * page + offset), -1 = skip
    state_slots: torch.Tensor        # [n_seqs] int32 recurrent-state slot of each sequence
    logit_rows: Optional[torch.Tensor] = None   # [R] int64 rows whose logits are wanted (None = all)
    max_q_len: int = 1
    max_ctx: int = 0
    write_state: bool = True         # recurrent layers advance their state (False for verify steps)
    embeds: Optional[torch.Tensor] = None       # input rows instead of the token embedding
    capture_layers: Optional[List[int]] = None  # layer outputs to return (EAGLE-3 features)
    cu_q_host: Optional[List[int]] = None
    decode_splits: Optional[int] = None
    replay: Optional[dict] = None                # verify steps: per-layer recurrent inputs kept for commit
    rope_table: Optional[torch.Tensor] = None    # [T, rot] per-token cos | sin rows (multi-section rotary positions of
    rope_rows: Optional[torch.Tensor] = None     #   image tokens); rope_rows = arange(T) indexes it like positions
    slots_ring: Optional[torch.Tensor] = None    # sliding-window layers with ring storage: their own KV cells [T] and
    block_table_ring: Optional[torch.Tensor] = None  #   block table (logical block j -> ring block j mod ring length)
    deepstack_rows: Optional[torch.Tensor] = None    # [R] int64 rows of this step that are image tokens, and per early
    deepstack: Optional[List[torch.Tensor]] = None   #   layer the [R, hidden] rows added to the stream after it

    @property
    def n_seqs(self) -> int:
        return self.ctx_lens.shape[0]


@dataclass
class StepOutput:
    hidden: torch.Tensor                     # [R, H] final-normed rows (logit rows)
    logits: Optional[torch.Tensor] = None    # [R, vocab] float32
    last_hidden: Optional[torch.Tensor] = None   # [T, H] residual stream before the final norm (MTP input)
    captures: Dict[int, torch.Tensor] = field(default_factory=dict)


class KvCache:
    """Per-layer paged K/V tensors ``[n_blocks, page, kv_heads, dim]`` (MLA layers: one latent row)."""

    def __init__(self, cfg: ModelConfig, n_blocks: int, page: int, device, dtype, kv_heads_local: Optional[int] = None,
                 extra_layers: int = 0, owns=None, ring_blocks: int = 0):
        """``ring_blocks`` > 0: sliding-window layers keep their K / V in a pool of that many blocks of their own
        (a short ring of blocks per sequence slot, ``engine.lm``) instead of ``n_blocks``."""
        self.page, self.n_blocks = page, n_blocks
        self.ring_blocks = ring_blocks
        self._kinds = tuple(cfg.layer_kinds)
        self.k: Dict[int, torch.Tensor] = {}
        self.v: Dict[int, torch.Tensor] = {}
        layers = [il for il in cfg.kv_layers() if owns is None or owns(il)]   # pipeline stage: own layers only
        kinds = {il: cfg.layer_kinds[il] for il in layers}
        for j in range(extra_layers):  # MTP blocks keep their own KV in the same block layout
            layers.append(cfg.n_layer + j)
            kinds[cfg.n_layer + j] = "mla" if cfg.kv_lora > 0 else "attn"
        for il in layers:
            if kinds[il] == "mla":
                self.k[il] = torch.zeros(n_blocks, page, 1, cfg.kv_lora + cfg.qk_rope_dim, device=device, dtype=dtype)
                self.v[il] = self.k[il]
            elif cfg.sandwich_norm and il < cfg.n_layer:
                if not cfg.owns_kv(il):
                    continue                          # reads its source layer's cache (mapped below)
                d, hk = cfg.attn_dims(il)
                nb = ring_blocks if (ring_blocks and kinds[il] == "swa") else n_blocks
                self.k[il] = torch.zeros(nb, page, hk, d, device=device, dtype=dtype)
                self.v[il] = torch.zeros(nb, page, hk, d, device=device, dtype=dtype)
            else:
                hk = kv_heads_local or cfg.n_kv_head
                nb = ring_blocks if (ring_blocks and kinds[il] == "swa") else n_blocks
                self.k[il] = torch.zeros(nb, page, hk, cfg.head_dim, device=device, dtype=dtype)
                self.v[il] = torch.zeros(nb, page, hk, cfg.head_dim, device=device, dtype=dtype)
        if cfg.sandwich_norm:
            for il in layers:
                if il < cfg.n_layer and not cfg.owns_kv(il):
                    src = cfg.kv_source(il)
                    self.k[il], self.v[il] = self.k[src], self.v[src]

    def bytes_per_block(self, swa_only: bool = False) -> int:
        """Bytes one block takes over every layer that owns a cache; ``swa_only`` counts the sliding-window layers
        alone (the part that moves into per-slot rings when ring storage is on)."""
        n = 0
        seen = set()
        kinds = self._kinds
        for il, k in self.k.items():
            if k.data_ptr() in seen:
                continue                              # a layer that reads another layer's cache
            seen.add(k.data_ptr())
            if swa_only and not (il < len(kinds) and kinds[il] == "swa"):
                continue
            n += k[0].numel() * k.element_size()
            if self.v[il] is not k:
                n += self.v[il][0].numel() * k.element_size()
        return n

    def copy_blocks(self, src: List[int], dst: List[int]):
        if not src:
            return
        s = torch.tensor(src, device=next(iter(self.k.values())).device)
        d = torch.tensor(dst, device=s.device)
        for il in self.k:
            self.k[il][d] = self.k[il][s]
            if self.v[il] is not self.k[il]:
                self.v[il][d] = self.v[il][s]


class StatePool:
    """Recurrent state in fixed slots: conv history + delta-rule / SSM state, float32
    (``src/model/core/state.rs:1297``)."""

    def __init__(self, cfg: ModelConfig, n_slots: int, device, tp: int = 1, owns=None):
        self.n_slots = n_slots
        self.conv: Dict[int, torch.Tensor] = {}
        self.ssm: Dict[int, torch.Tensor] = {}
        for il in cfg.recurrent_layers():
            if owns is not None and not owns(il):
                continue
            kind = cfg.layer_kinds[il]
            if kind == "gdn":
                C = cfg.gdn_conv_channels() // tp
                self.conv[il] = torch.zeros(n_slots, C, cfg.gdn_conv - 1, device=device, dtype=torch.float32)
                self.ssm[il] = torch.zeros(n_slots, cfg.gdn_v_heads // tp, cfg.gdn_k_dim, cfg.gdn_v_dim, device=device,
                                           dtype=torch.float32)
            elif kind == "kda":
                c = cfg.kda_heads * cfg.kda_head_dim
                self.conv[il] = torch.zeros(n_slots, 3 * c, cfg.kda_conv - 1, device=device, dtype=torch.float32)
                # state[head, value row j, key channel i]
                self.ssm[il] = torch.zeros(n_slots, cfg.kda_heads, cfg.kda_head_dim, cfg.kda_head_dim, device=device,
                                           dtype=torch.float32)
            elif kind == "mamba2":
                di = cfg.ssm_heads * cfg.ssm_head_dim
                C = di + 2 * cfg.ssm_groups * cfg.ssm_state
                self.conv[il] = torch.zeros(n_slots, C, cfg.ssm_conv - 1, device=device, dtype=torch.float32)
                self.ssm[il] = torch.zeros(n_slots, cfg.ssm_heads, cfg.ssm_head_dim, cfg.ssm_state, device=device,
                                           dtype=torch.float32)

    def attach_rings(self, kv: "KvCache", ring_len: int, layers) -> None:
        """Sliding-window rings are per-slot state too: slot s owns ring blocks [s * ring_len, (s + 1) * ring_len) of
        the given layers' K / V pools, so a snapshot of a slot carries its window history (the reference's ring
        checkpoints, ``src/engine/ring_checkpoints.rs``) and a prefix-cache hit can resume from it."""
        self.ring_len = ring_len
        self.rings = [(kv.k[il], kv.v[il]) for il in layers]

    def _ring_views(self, slot: int):
        L = getattr(self, "ring_len", 0)
        for k, v in getattr(self, "rings", ()):
            yield k[slot * L:(slot + 1) * L]
            if v is not k:
                yield v[slot * L:(slot + 1) * L]

    def clear(self, slot: int):
        for t in list(self.conv.values()) + list(self.ssm.values()):
            t[slot].zero_()

    def copy(self, src: int, dst: int):
        for t in list(self.conv.values()) + list(self.ssm.values()):
            t[dst].copy_(t[src])
        for a, b in zip(self._ring_views(src), self._ring_views(dst)):
            b.copy_(a)

    def bytes_per_slot(self) -> int:
        n = sum(t[0].numel() * 4 for t in list(self.conv.values()) + list(self.ssm.values()))
        return n + sum(t.numel() * t.element_size() for t in self._ring_views(0))


def fold_shared_expert(w: Dict[str, object], p: str, cfg: ModelConfig) -> bool:
    """Stacks the shared expert of layer ``p`` behind the routed experts: ``{p}.moe.gate_up_s`` / ``down_s`` hold
    E + 1 groups, and ``gate_up`` / ``down`` / ``sh_gate_up`` / ``sh_down`` become views of them (so prompt-sized
    steps, which run the shared expert as a dense FFN, share the storage). Plain bf16 tensors only: quantise after
    folding."""
    gu, dn = w.get(f"{p}.moe.gate_up"), w.get(f"{p}.moe.down")
    sgu, sdn = w.get(f"{p}.moe.sh_gate_up"), w.get(f"{p}.moe.sh_down")
    if (not isinstance(gu, torch.Tensor) or not isinstance(sgu, torch.Tensor) or f"{p}.moe.gate_up_s" in w
            or not gu.is_cuda or sgu.shape[0] != gu.shape[1] or sdn.shape[1] != dn.shape[2]):
        return False
    E = gu.shape[0]
    gus = torch.empty(E + 1, *gu.shape[1:], dtype=gu.dtype, device=gu.device)
    gus[:E].copy_(gu)
    gus[E].copy_(sgu)
    del gu
    w[f"{p}.moe.gate_up"] = None
    dns = torch.empty(E + 1, *dn.shape[1:], dtype=dn.dtype, device=dn.device)
    dns[:E].copy_(dn)
    dns[E].copy_(sdn)
    w[f"{p}.moe.gate_up_s"], w[f"{p}.moe.down_s"] = gus, dns
    w[f"{p}.moe.gate_up"], w[f"{p}.moe.down"] = gus[:E], dns[:E]
    w[f"{p}.moe.sh_gate_up"], w[f"{p}.moe.sh_down"] = gus[E], dns[E]
    return True


def place_shared_expert(w: Dict[str, object], p: str, il: int, cfg: ModelConfig, rank: int, world: int) -> bool:
    """Several ranks with whole (unsliced) shared experts: rank ``il % world`` keeps the shared expert of layer
    ``il`` and stacks it behind its local routed experts (``fold_shared_expert``); the other ranks drop it, so the
    layer's reduction sums exactly one copy. Returns whether this rank keeps it."""
    if world <= 1 or il % world == rank:
        fold_shared_expert(w, p, cfg)
        return True
    for k in ("sh_gate_up", "sh_down", "sh_gate"):
        w.pop(f"{p}.moe.{k}", None)
    return False


def quantize_moe_layer_nvfp4(w: Dict[str, object], p: str, native: bool = True) -> int:
    """NVFP4-encodes the expert tensors of MoE layer ``p`` in place (stacked form when the shared expert was
    folded in, else the routed experts and the shared expert separately). Returns the bytes saved."""
    from ..ops.sm100 import Nv4Weight, QWeight
    cls = Nv4Weight if native else QWeight
    saved = 0

    def enc(t, dual):
        nonlocal saved
        rows, K = t.shape[-2], t.shape[-1]
        ok = isinstance(t, torch.Tensor) and t.dtype == torch.bfloat16 and K % 256 == 0 and rows % 128 == 0 and \
            (not dual or (rows // 2) % 128 == 0)
        if not ok:
            return None
        saved += t.numel() * 2 - t.numel() * 9 // 16
        return cls.quantize_cuda(t, dual_rows=rows // 2 if dual else 0)

    if f"{p}.moe.gate_up_s" in w:
        gus, dns = w[f"{p}.moe.gate_up_s"], w[f"{p}.moe.down_s"]
        if not isinstance(gus, torch.Tensor):
            return 0
        E = gus.shape[0] - 1
        for k in ("gate_up", "down", "sh_gate_up", "sh_down"):
            w[f"{p}.moe.{k}"] = None
        qg, qd = enc(gus, True), enc(dns, False)
        if qg is None or qd is None:
            w[f"{p}.moe.gate_up"], w[f"{p}.moe.down"] = gus[:E], dns[:E]
            w[f"{p}.moe.sh_gate_up"], w[f"{p}.moe.sh_down"] = gus[E], dns[E]
            return 0
        w[f"{p}.moe.gate_up_s"], w[f"{p}.moe.down_s"] = qg, qd
        w[f"{p}.moe.gate_up"], w[f"{p}.moe.down"] = qg.narrow(0, E), qd.narrow(0, E)
        w[f"{p}.moe.sh_gate_up"] = qg.narrow(E, E + 1).squeeze0()
        w[f"{p}.moe.sh_down"] = qd.narrow(E, E + 1).squeeze0()
        return saved
    for k, dual in (("gate_up", True), ("down", False), ("sh_gate_up", True), ("sh_down", False)):
        t = w.get(f"{p}.moe.{k}")
        if isinstance(t, torch.Tensor):
            q = enc(t, dual)
            if q is not None:
                w[f"{p}.moe.{k}"] = q
    return saved


def quantize_moe_layer_fp8(w: Dict[str, object], p: str) -> int:
    """Block-scaled FP8 encoding of the expert tensors of MoE layer ``p`` in place (the stacked form when the shared
    expert was folded in, else the routed experts and the shared expert separately). Returns the bytes saved."""
    from ..ops.sm100 import Fp8Weight
    saved = 0

    def ok(t, dual):
        return (isinstance(t, torch.Tensor) and t.dtype == torch.bfloat16 and t.is_cuda and t.shape[-1] % 128 == 0
                and t.shape[-2] % 128 == 0 and (not dual or (t.shape[-2] // 2) % 128 == 0))

    if f"{p}.moe.gate_up_s" in w:
        gus, dns = w[f"{p}.moe.gate_up_s"], w[f"{p}.moe.down_s"]
        if not ok(gus, True) or not ok(dns, False):
            return 0
        E = gus.shape[0] - 1
        for k in ("gate_up", "down", "sh_gate_up", "sh_down"):
            w[f"{p}.moe.{k}"] = None                 # views of the bf16 stacks
        saved = gus.numel() + dns.numel()
        qg, qd = Fp8Weight.quantize(gus), Fp8Weight.quantize(dns)
        w[f"{p}.moe.gate_up_s"], w[f"{p}.moe.down_s"] = qg, qd
        w[f"{p}.moe.gate_up"], w[f"{p}.moe.down"] = qg.narrow(0, E), qd.narrow(0, E)
        w[f"{p}.moe.sh_gate_up"] = qg.narrow(E, E + 1).squeeze0()
        w[f"{p}.moe.sh_down"] = qd.narrow(E, E + 1).squeeze0()
        return saved
    for k, dual in (("gate_up", True), ("down", False), ("sh_gate_up", True), ("sh_down", False)):
        t = w.get(f"{p}.moe.{k}")
        if ok(t, dual):
            w[f"{p}.moe.{k}"] = Fp8Weight.quantize(t)
            saved += t.numel()
    return saved


class Decoder:
    """Weights + forward. ``weights`` uses the canonical names of ``models.weights``."""

    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], pctx: Optional[ParallelCtx] = None,
                 max_position: Optional[int] = None, pipe=None):
        self.cfg = cfg
        if cfg.hyper_streams > 1 and pipe is not None:
            raise NotImplementedError("hyper-connection models run without pipeline stages")
        self.w = weights
        self.pctx = pctx or ParallelCtx.single()
        self.pipe = pipe          # parallel.pipeline.PipeStage: this rank runs layers [pipe.lo, pipe.hi)
        dev = weights["tok_embd"].device
        self.device = dev
        self.dtype = weights["tok_embd"].dtype
        mp = max_position or cfg.max_position
        scaling = cfg.rope_scaling
        if cfg.rope_freq_factors:
            scaling = {"type": "factors", "factors": list(cfg.rope_freq_factors)}
        self.cos_sin = ops.reference.rope_cos_sin(mp, cfg.rope_dim, cfg.rope_theta, scaling, device=dev)
        self.cos_sin_swa = None
        if cfg.sandwich_norm and (cfg.rope_theta_swa or cfg.swa_head_dim):
            # sliding-window layers rotate their (own-sized) heads whole with a base of their own
            self.cos_sin_swa = ops.reference.rope_cos_sin(mp, cfg.swa_head_dim or cfg.head_dim,
                                                          cfg.rope_theta_swa or cfg.rope_theta, None, device=dev)
        tp = self.pctx.tp
        self.n_head_l = cfg.n_head // tp
        self.n_kv_l = max(1, cfg.n_kv_head // tp)
        self.gdn_k_l = max(1, cfg.gdn_k_heads // tp)
        self.gdn_v_l = max(1, cfg.gdn_v_heads // tp)
        self.lm_head = weights.get("output", weights["tok_embd"])
        self.head_split = None            # (first row, rows) of this rank's slice of the vocabulary (split_head)
        self.expert_cache: Dict[str, object] = {}     # layer prefix -> residency.ExpertCache (offload modes)
        self._mla_uk: Dict[str, torch.Tensor] = {}    # layer prefix -> W_uk^T per head (absorb projection, K-major)

    def offload_experts(self, n_slots: int, profile: Optional[dict] = None, ssd_dir: Optional[str] = None,
                        ram_experts: int = 0):
        """Moves every MoE layer's routed experts to pinned host memory behind ``n_slots`` HBM slots; with
        ``ssd_dir`` to one file per layer in that directory, behind ``ram_experts`` experts per layer in host
        memory and the HBM slots."""
        import os
        from ..residency.experts import ExpertCache
        if ssd_dir:
            os.makedirs(ssd_dir, exist_ok=True)
        for il in range(self.cfg.n_layer):
            if not self.cfg.is_moe_layer(il):
                continue
            p = f"l{il}"
            gu, dn = self.w.pop(f"{p}.moe.gate_up"), self.w.pop(f"{p}.moe.down")
            self.expert_cache[p] = ExpertCache(gu, dn, n_slots, self.device, profile=(profile or {}).get(p),
                                               ssd_path=os.path.join(ssd_dir, f"{p}.experts.bin") if ssd_dir else None,
                                               ram_experts=ram_experts)

    def quantize_experts_nvfp4(self, native: bool = True) -> int:
        """Re-encodes the routed experts (and the shared expert) of every MoE layer to NVFP4 in place: 3.5x less
        HBM for the bulk of a MoE model. ``native``: the layout of the block-scaled tensor-core GEMM
        (``ops.sm100.Nv4Weight``: activations are quantised to NVFP4 too and nothing is expanded); otherwise the
        grouped GEMM streams the 4-bit codes and expands them inside the kernel (``ops.sm100.QWeight``).
        Returns the number of bytes saved. GPU only."""
        saved = 0
        for il in range(self.cfg.n_layer):
            if self.cfg.is_moe_layer(il):
                saved += quantize_moe_layer_nvfp4(self.w, f"l{il}", native)
        return saved

    def fold_shared_experts(self) -> int:
        """Stacks every MoE layer's shared expert behind its routed experts (when both have the same width) so that
        decode-sized steps run it as one more slot of the grouped GEMMs instead of three launches of its own.
        Returns the number of layers folded."""
        n = 0
        for il in range(self.cfg.n_layer):
            if self.cfg.is_moe_layer(il) and fold_shared_expert(self.w, f"l{il}", self.cfg):
                n += 1
        return n

    FP8_LEAVES = ("attn.qkv", "attn.o", "mlp.gate_up", "mlp.down", "moe.gate_up", "moe.down", "moe.sh_gate_up",
                  "moe.sh_down", "mla.q_a", "mla.q_b", "mla.q", "mla.kv_a", "mla.o", "gdn.in_qkv", "gdn.in_z", "gdn.out")

    def quantize_weights_fp8(self, experts_only: bool = False, ffn_only: bool = False) -> int:
        """Re-encodes the projection weights (routed experts, dense and shared FFNs, attention / latent-attention /
        linear-attention projections) to block-scaled FP8 in place: e4m3 with one fp32 scale per 128 x 128 block,
        the encoding of FP8 checkpoints. The GEMMs then run on the e4m3 tensor-core path with activations
        quantised per token and 128 columns (``ops.sm100.Fp8Weight``). Embedding, head, router, norms and the small
        gate projections stay as they are; ``ffn_only`` also leaves the attention projections alone (they are a
        few per cent of the bytes, and a decode step then has no activation encoding in front of them).
        Returns the number of bytes saved. GPU only."""
        from ..ops.sm100 import Fp8Weight
        saved = 0
        for name in list(self.w):
            t = self.w[name]
            leaf = name.split(".", 1)[1] if "." in name else name
            if leaf not in self.FP8_LEAVES or not isinstance(t, torch.Tensor) or t.dtype != torch.bfloat16:
                continue
            if experts_only and leaf not in ("moe.gate_up", "moe.down"):
                continue
            if ffn_only and not leaf.startswith(("mlp.", "moe.")):
                continue
            rows, K = t.shape[-2], t.shape[-1]
            if K % 128 or rows % 128:
                continue
            if leaf.endswith("gate_up") and (rows // 2) % 128:
                continue                      # the gate and the up half must start on block boundaries
            self.w[name] = Fp8Weight.quantize(t)
            saved += t.numel()
            del t
        return saved

    # ------------------------------------------------------------------ blocks
    def _attn(self, p: str, il: int, x, b: StepBatch, kv: KvCache, window: int, rope: bool = True):
        cfg, w = self.cfg, self.w
        D = cfg.head_dim
        qkv = ops.linear(x, w[f"{p}.attn.qkv"])
        cos_sin, positions = (self.cos_sin, b.positions) if b.rope_table is None else (b.rope_table, b.rope_rows)
        slots, table = b.slots, b.block_table
        if window > 0 and b.slots_ring is not None:
            slots, table = b.slots_ring, b.block_table_ring      # this layer's K / V live in the sequence's ring
        q, gate = ops.qk_norm_rope_append(qkv, self.n_head_l, self.n_kv_l, D, w.get(f"{p}.attn.q_norm"),
                                          w.get(f"{p}.attn.k_norm"), cfg.rms_eps, cfg.norm_offset, cos_sin,
                                          cfg.rope_dim if rope else 0, positions, slots, kv.k[il], kv.v[il],
                                          cfg.gated_attn)
        scale = cfg.attn_scale or D ** -0.5
        o = ops.paged_attention(q, kv.k[il], kv.v[il], table, b.ctx_lens, b.cu_q, b.max_q_len, scale,
                                window=window, decode_splits=b.decode_splits, max_ctx=b.max_ctx or None)
        if cfg.gated_attn:
            o = ops.apply_output_gate(o, gate, self.n_head_l, D)
        return self.pctx.defer_linear(o.reshape(o.shape[0], -1), w[f"{p}.attn.o"], lazy=True)

    def _gdn(self, p: str, il: int, x, b: StepBatch, st: StatePool):
        cfg, w = self.cfg, self.w
        nk, nv, dk, dv = self.gdn_k_l, self.gdn_v_l, cfg.gdn_k_dim, cfg.gdn_v_dim
        w_all = w.get(f"{p}.gdn.in_all")
        if w_all is not None:
            # one GEMM for the three input projections; the pieces are column slices of its output
            C = 2 * nk * dk + nv * dv
            proj = ops.linear(x, w_all)
            if (x.is_cuda and b.max_q_len == 1 and b.write_state and b.replay is None
                    and proj.shape[0] == b.state_slots.shape[0] and ops.sm100.gdn_decode_fused_ok(nk, nv, dk, dv, cfg.gdn_conv)):
                # decode step: conv, gates, delta rule and gated norm in one launch
                n = ops.sm100.gdn_decode_fused(proj, w[f"{p}.gdn.conv_w"], st.conv[il], w[f"{p}.gdn.A"],
                                               w[f"{p}.gdn.dt_bias"], w[f"{p}.gdn.norm"], cfg.rms_eps, cfg.gdn_gate_act,
                                               st.ssm[il], b.state_slots, nk, nv, dk, dv, cfg.gdn_tiled_heads,
                                               dk ** -0.5, 1e-6)
                return self.pctx.defer_linear(n, w[f"{p}.gdn.out"], lazy=True)
            mixed, z, ba = proj[:, :C], proj[:, C:C + nv * dv], proj[:, C + nv * dv:]
        else:
            mixed = ops.linear(x, w[f"{p}.gdn.in_qkv"])
            z = ops.linear(x, w[f"{p}.gdn.in_z"])
            ba = ops.linear(x, w[f"{p}.gdn.in_ba"])
        conv = ops.causal_conv1d_silu(mixed, w[f"{p}.gdn.conv_w"], None, st.conv[il], b.cu_q, b.state_slots,
                                      write_state=b.write_state, max_len=b.max_q_len)
        g, beta = ops.gdn_gates(ba[:, nv:], ba[:, :nv], w[f"{p}.gdn.A"], w[f"{p}.gdn.dt_bias"])
        if b.replay is not None:
            b.replay[il] = (mixed, g, beta)
        o = ops.gdn_recurrent(conv, g, beta, st.ssm[il], b.cu_q, b.state_slots, nk, nv, dk, dv, cfg.gdn_tiled_heads,
                              dk ** -0.5, 1e-6, write_state=b.write_state, cu_host=b.cu_q_host)
        n = ops.gated_rmsnorm(o, z, w[f"{p}.gdn.norm"], cfg.rms_eps, cfg.gdn_gate_act)
        return self.pctx.defer_linear(n.reshape(n.shape[0], -1), w[f"{p}.gdn.out"], lazy=True)

    def fuse_gdn_in_proj(self) -> int:
        """Stacks the three input projections of every Gated DeltaNet layer (q/k/v, z, b/a) into one weight
        ``gdn.in_all`` so that a layer needs one GEMM for them; the separate names stay as views of its rows.
        Returns the number of layers fused."""
        n = 0
        for il in self.cfg.recurrent_layers():
            p = f"l{il}"
            parts = [self.w.get(f"{p}.gdn.{k}") for k in ("in_qkv", "in_z", "in_ba")]
            if f"{p}.gdn.in_all" in self.w or any(not isinstance(t, torch.Tensor) or t.dtype != torch.bfloat16 for t in parts):
                continue
            allw = torch.cat(parts, 0)
            r0 = 0
            for k, t in zip(("in_qkv", "in_z", "in_ba"), parts):
                self.w[f"{p}.gdn.{k}"] = allw[r0:r0 + t.shape[0]]
                r0 += t.shape[0]
            del parts
            self.w[f"{p}.gdn.in_all"] = allw
            n += 1
        return n

    def fuse_mla_in_proj(self) -> int:
        """Stacks the two input projections of every latent-attention layer that read the layer input (the low-rank
        query projection ``q_a`` and the latent / rope-key projection ``kv_a``) into one weight ``mla.qkv_a`` so that
        a layer needs one GEMM for them (bf16 weights only). Returns the number of layers fused."""
        n = 0
        for il, kind in enumerate(self.cfg.layer_kinds):
            p = f"l{il}"
            qa, kva = self.w.get(f"{p}.mla.q_a"), self.w.get(f"{p}.mla.kv_a")
            if kind != "mla" or f"{p}.mla.qkv_a" in self.w or not isinstance(qa, torch.Tensor) or \
                    not isinstance(kva, torch.Tensor) or qa.dtype != torch.bfloat16 or kva.dtype != torch.bfloat16 or \
                    not qa.is_cuda or qa.shape[0] % 8:
                continue
            both = torch.cat([qa, kva], 0)
            self.w[f"{p}.mla.q_a"], self.w[f"{p}.mla.kv_a"] = both[:qa.shape[0]], both[qa.shape[0]:]
            self.w[f"{p}.mla.qkv_a"] = both
            n += 1
        return n

    def absorb_mla_q(self) -> int:
        """Folds the key up-projection of every latent-attention layer into its query projection for decode-sized
        steps: ``mla.q_b_abs`` [heads * (kv_lora + rope), q_lora] maps the normalised low-rank query straight to
        the absorbed query rows the attention kernel reads ([q_nope W_uk | q_pe] per head), so a decode step needs
        no per-head absorb GEMM. The folded weight is (kv_lora + rope) / (nope + rope) times the size of ``q_b``
        and costs that much more arithmetic, so prompt-sized steps keep the two-step form. Returns the number of
        layers folded (bf16 weights with a low-rank query only)."""
        cfg, n = self.cfg, 0
        L, dn, dr, dvh = cfg.kv_lora, cfg.qk_nope_dim, cfg.qk_rope_dim, cfg.v_head_dim
        for il, kind in enumerate(cfg.layer_kinds):
            p = f"l{il}"
            qb, kvb = self.w.get(f"{p}.mla.q_b"), self.w.get(f"{p}.mla.kv_b")
            if kind != "mla" or cfg.q_lora <= 0 or f"{p}.mla.q_b_abs" in self.w or not isinstance(qb, torch.Tensor) \
                    or not isinstance(kvb, torch.Tensor) or qb.dtype != torch.bfloat16 or not qb.is_cuda:
                continue
            nh = qb.shape[0] // (dn + dr)
            qb3 = qb.view(nh, dn + dr, cfg.q_lora)
            w_uk = kvb.view(nh, dn + dvh, L)[:, :dn]                                    # [heads, nope, kv_lora]
            nope = torch.bmm(w_uk.transpose(1, 2).float(), qb3[:, :dn].float())        # [heads, kv_lora, q_lora]
            self.w[f"{p}.mla.q_b_abs"] = torch.cat([nope.to(qb.dtype), qb3[:, dn:]], 1).reshape(nh * (L + dr), cfg.q_lora)
            n += 1
        return n

    def _mla(self, p: str, il: int, x, b: StepBatch, kv: KvCache):
        """Latent attention: cache row = [rmsnorm(c_kv) | rope(k_pe)]; keys/values are expanded from
        the cached latents of each sequence (prefill form), queries carry [nope | rope] parts."""
        cfg, w = self.cfg, self.w
        nh, dn, dr, dvh, L = self.n_head_l, cfg.qk_nope_dim, cfg.qk_rope_dim, cfg.v_head_dim, cfg.kv_lora
        T = x.shape[0]
        kva = None
        both_w = w.get(f"{p}.mla.qkv_a")
        if cfg.q_lora > 0:
            if both_w is not None and x.is_cuda:
                both = ops.linear(x, both_w)            # q_a and kv_a in one GEMM; the parts are column slices
                qa, kva = both[:, :cfg.q_lora], both[:, cfg.q_lora:]
            else:
                qa = ops.linear(x, w[f"{p}.mla.q_a"])
            qa, _ = ops.rmsnorm(qa, w[f"{p}.mla.q_a_norm"], cfg.rms_eps, cfg.norm_offset)
            qb_abs = w.get(f"{p}.mla.q_b_abs")
            if (qb_abs is not None and T <= 64 and x.is_cuda and x.dtype == torch.bfloat16
                    and ops.sm100.mla_supported(nh, L, dr, kv.page)):
                # decode-sized step: one GEMM gives the absorbed query rows; their rope part is rotated in place
                q_abs = ops.linear(qa, qb_abs).view(T, nh, L + dr)
                if kva is None:
                    kva = ops.linear(x, w[f"{p}.mla.kv_a"])
                ops.sm100.mla_prep(kva, w[f"{p}.mla.kv_a_norm"], cfg.rms_eps, cfg.norm_offset, q_abs, L, self.cos_sin,
                                   b.positions, b.slots, kv.k[il], q_abs)
                return self._mla_tail(p, il, q_abs, b, kv, True)
            q = ops.linear(qa, w[f"{p}.mla.q_b"])
        else:
            q = ops.linear(x, w[f"{p}.mla.q"])
        q = q.view(T, nh, dn + dr)
        if kva is None:
            kva = ops.linear(x, w[f"{p}.mla.kv_a"])
        wkv_b = w[f"{p}.mla.kv_b"].view(nh, dn + dvh, L)
        if x.is_cuda and x.dtype == torch.bfloat16 and ops.sm100.mla_supported(nh, L, dr, kv.page):
            # absorbed form on the tensor cores: q_abs = [q_nope W_uk | rope(q_pe)], o = (softmax . c_kv) W_uv
            q_abs = torch.empty(T, nh, L + dr, dtype=x.dtype, device=x.device)
            own = (ops.sm100.TUNE["mla_head_gemm"] and dn % 64 == 0 and dvh % 8 == 0 and (dn + dr) % 8 == 0
                   and isinstance(w[f"{p}.mla.kv_b"], torch.Tensor))
            if own:
                # per-head absorb and value projections on the grouped tcgen05 GEMM (group = head), each head's
                # slice read and written in place
                uk = self._mla_uk.get(p)
                if uk is None:
                    uk = wkv_b[:, :dn].transpose(1, 2).contiguous().view(nh * L, dn)     # W_uk^T per head, K-major
                    self._mla_uk[p] = uk
                ops.sm100.head_linear(q.view(T, nh * (dn + dr)), uk, nh, L, L, dn, dn + dr, q_abs.view(T * nh, L + dr))
            else:
                q_abs[..., :L] = torch.bmm(q[..., :dn].transpose(0, 1), wkv_b[:, :dn]).transpose(0, 1)
            ops.sm100.mla_prep(kva, w[f"{p}.mla.kv_a_norm"], cfg.rms_eps, cfg.norm_offset, q, dn, self.cos_sin,
                               b.positions, b.slots, kv.k[il], q_abs)
            return self._mla_tail(p, il, q_abs, b, kv, own)
        return self._mla_reference(p, il, x, q, kva, b, kv)

    def _mla_tail(self, p: str, il: int, q_abs, b: StepBatch, kv: KvCache, own: bool):
        """Latent attention over the absorbed query rows, the per-head value projection and the output projection."""
        cfg, w = self.cfg, self.w
        T, nh = q_abs.shape[0], q_abs.shape[1]
        L, dn, dvh = cfg.kv_lora, cfg.qk_nope_dim, cfg.v_head_dim
        scale = cfg.attn_scale or (dn + cfg.qk_rope_dim) ** -0.5
        o_lat = ops.sm100.mla_attn(q_abs, kv.k[il], b.cu_q, b.ctx_lens, b.block_table, kv.page, b.max_q_len, scale,
                                   max_ctx=b.max_ctx or None)
        if own and isinstance(w[f"{p}.mla.kv_b"], torch.Tensor) and dvh % 8 == 0 and ops.sm100.TUNE["mla_head_gemm"]:
            out = torch.empty(T, nh * dvh, dtype=q_abs.dtype, device=q_abs.device)
            w_uv = w[f"{p}.mla.kv_b"].view(nh * (dn + dvh), L)[dn:]                       # head h: rows h*(dn+dvh)..+dvh
            ops.sm100.head_linear(o_lat.view(T, nh * L), w_uv, nh, dn + dvh, dvh, L, L, out.view(T * nh, dvh))
        else:
            wkv_b = w[f"{p}.mla.kv_b"].view(nh, dn + dvh, L)
            out = torch.bmm(o_lat.transpose(0, 1), wkv_b[:, dn:].transpose(1, 2)).transpose(0, 1)
        return ops.linear(out.reshape(T, nh * dvh), w[f"{p}.mla.o"])

    def _mla_reference(self, p: str, il: int, x, q, kva, b: StepBatch, kv: KvCache):
        """Latent attention in plain tensor operations (CPU ranks, shapes the kernels do not take)."""
        cfg, w = self.cfg, self.w
        nh = self.n_head_l
        dn, dr, dvh, L = cfg.qk_nope_dim, cfg.qk_rope_dim, cfg.v_head_dim, cfg.kv_lora
        T = x.shape[0]
        wkv_b = w[f"{p}.mla.kv_b"].view(nh, dn + dvh, L)
        scale = cfg.attn_scale or (dn + dr) ** -0.5
        ckv, _ = ops.rmsnorm(kva[:, :L].contiguous(), w[f"{p}.mla.kv_a_norm"], cfg.rms_eps, cfg.norm_offset)
        k_pe = ops.reference.apply_rope(kva[:, L:].reshape(T, 1, dr), self.cos_sin, b.positions, dr)
        q_pe = ops.reference.apply_rope(q[..., dn:], self.cos_sin, b.positions, dr)
        row = torch.cat([ckv, k_pe.reshape(T, dr)], dim=-1).to(kv.k[il].dtype)
        valid = b.slots >= 0
        kv.k[il].view(-1, L + dr)[b.slots[valid]] = row[valid]
        out = torch.empty(T, nh, dvh, device=x.device, dtype=x.dtype)
        cu = b.cu_q_host if b.cu_q_host is not None else b.cu_q.tolist()
        ctxs = b.ctx_lens.tolist()
        page = kv.page
        for i in range(b.n_seqs):
            q0, q1 = cu[i], cu[i + 1]
            if q1 <= q0:
                continue
            ctx = ctxs[i]
            nb = (ctx + page - 1) // page
            lat = kv.k[il][b.block_table[i, :nb].long()].reshape(-1, L + dr)[:ctx].float()
            c, kp = lat[:, :L], lat[:, L:]
            # absorbed form: scores = (q_nope W_uk) . c + q_pe . k_pe ; out = (p . c) W_uv
            q_abs = torch.einsum("qhd,hdl->qhl", q[q0:q1, :, :dn].float(), wkv_b[:, :dn].float())
            s = (torch.einsum("qhl,kl->hqk", q_abs, c) + torch.einsum("qhd,kd->hqk", q_pe[q0:q1].float(), kp)) * scale
            qpos = torch.arange(ctx - (q1 - q0), ctx, device=x.device)[:, None]
            kpos = torch.arange(ctx, device=x.device)[None, :]
            s = s.masked_fill((kpos > qpos)[None], float("-inf"))
            pr = torch.softmax(s, dim=-1)
            o_lat = torch.einsum("hqk,kl->qhl", pr, c)
            out[q0:q1] = torch.einsum("qhl,hvl->qhv", o_lat, wkv_b[:, dn:].float()).to(x.dtype)
        return ops.linear(out.reshape(T, nh * dvh), w[f"{p}.mla.o"])

    def _kda(self, p: str, il: int, x, b: StepBatch, st: StatePool):
        """Kimi delta attention (``src/model/glm5next.rs::glm_kda_on``, ``ops.rs::cpu_kda_scan`` in the reference):
        q, k, v each through a causal short convolution and SiLU; a per-channel log decay
        ``lower * sigmoid(-(f_b f_a x + dt_bias) * A)``; the gated delta rule over a [d, d] state per head
        (row j of the state decays per key channel, then moves by beta * (v_j - row . k) along k); an RMS norm
        gated by ``sigmoid(g_b g_a x)``; the output projection. Tensor operations on every back-end: the token
        recurrence is a loop over the step's longest sequence with all sequences and heads batched (a decode step
        is one iteration)."""
        cfg, w = self.cfg, self.w
        nh, d, KC = cfg.kda_heads, cfg.kda_head_dim, cfg.kda_conv
        c = nh * d
        T = x.shape[0]
        f32 = torch.float32
        qkv = ops.linear(x, w[f"{p}.kda.qkv"]).to(f32)                                   # [T, 3c]
        z = ops.linear(ops.linear(x, w[f"{p}.kda.f_a"]), w[f"{p}.kda.f_b"]).to(f32)      # [T, c]
        A = w[f"{p}.kda.A"].to(f32).repeat_interleave(d)
        g = cfg.kda_lower * torch.sigmoid(-((z + w[f"{p}.kda.dt_bias"].to(f32)) * A))    # log decay per channel
        beta = torch.sigmoid(ops.linear(x, w[f"{p}.kda.beta"]).to(f32))                  # [T, heads]
        gate = ops.linear(ops.linear(x, w[f"{p}.kda.g_a"]), w[f"{p}.kda.g_b"]).to(f32)   # [T, c]
        cw = w[f"{p}.kda.conv_w"].to(f32)                                                # [3c, KC]
        cu = b.cu_q_host if b.cu_q_host is not None else b.cu_q.tolist()
        n_seq = len(cu) - 1
        slots = b.state_slots.long()
        lens = [cu[i + 1] - cu[i] for i in range(n_seq)]
        L = max(lens) if lens else 0
        # rows of the step as [sequence, time] with padding: index T is a zero row
        idx = torch.full((n_seq, L), T, dtype=torch.int64)
        for i in range(n_seq):
            idx[i, :lens[i]] = torch.arange(cu[i], cu[i + 1])
        idx = idx.to(x.device)
        live = idx < T                                                                   # [n_seq, L]
        pad = lambda t: torch.cat([t, t.new_zeros(1, *t.shape[1:])], 0)[idx]             # noqa: E731
        xs, gs, bs = pad(qkv), pad(g), pad(beta)                                         # [n_seq, L, ...]
        hist = st.conv[il][slots]                                                        # [n_seq, 3c, KC - 1]
        S = st.ssm[il][slots]                                                            # [n_seq, heads, d(j), d(i)]
        out = torch.zeros(n_seq, L, c, dtype=f32, device=x.device)
        qs = d ** -0.5
        for t in range(L):
            m = live[:, t]
            xt = xs[:, t]                                                                # [n_seq, 3c]
            win = torch.cat([hist, xt.unsqueeze(2)], 2)                                  # [n_seq, 3c, KC]
            y = (win * cw.unsqueeze(0)).sum(2)
            y = y * torch.sigmoid(y)
            hist = torch.where(m[:, None, None], win[:, :, 1:], hist)
            q, k, v = (y[:, j * c:(j + 1) * c].view(n_seq, nh, d) for j in range(3))
            qn = q * (qs * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6))
            kn = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
            dec = gs[:, t].view(n_seq, nh, d).exp()                                      # per key channel
            S2 = S * dec.unsqueeze(2)
            delta = (v - torch.einsum("shji,shi->shj", S2, kn)) * bs[:, t].unsqueeze(-1)
            S2 = S2 + delta.unsqueeze(-1) * kn.unsqueeze(2)
            out[:, t] = torch.einsum("shji,shi->shj", S2, qn).reshape(n_seq, c)
            S = torch.where(m[:, None, None, None], S2, S)
        if b.write_state:
            st.conv[il][slots] = hist
            st.ssm[il][slots] = S
        o = out[live]                                                                    # back to step order
        o = o.view(T, nh, d)
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * w[f"{p}.kda.norm"].to(f32)
        o = o * torch.sigmoid(gate.view(T, nh, d))
        return ops.linear(o.reshape(T, c).to(x.dtype), w[f"{p}.kda.out"])

    # ------------------------------------------------------------------ Gemma-4 layer form
    def _gemma_attn(self, p: str, il: int, h, b: StepBatch, kv: KvCache):
        """Attention of a Gemma-4 layer (``src/model/gemma4.rs::gemma4_attend_qkv`` in the reference): head size,
        kv-head count and rotary table by layer kind; q and k RMS-normed with weights, v without; a global layer
        without a value projection uses its raw keys as values; a layer that owns no cache reads its source layer's;
        attention is unscaled."""
        cfg, w = self.cfg, self.w
        kind = cfg.layer_kinds[il]
        D, n_kv = cfg.attn_dims(il)
        nh = cfg.n_head
        T = h.shape[0]
        swa = kind == "swa"
        cos_sin = self.cos_sin_swa if (swa and self.cos_sin_swa is not None) else self.cos_sin
        rot = D if swa else cfg.rope_dim
        proj = ops.linear(h, w[f"{p}.attn.qkv"])
        slots, table = b.slots, b.block_table
        if swa and b.slots_ring is not None:
            slots, table = b.slots_ring, b.block_table_ring
        if cfg.owns_kv(il):
            q, k = proj[:, :nh * D], proj[:, nh * D:(nh + n_kv) * D]
            v = proj[:, (nh + n_kv) * D:] if cfg.has_v_proj(il) else k
            if cfg.v_norm:
                vf = v.reshape(T, n_kv, D).float()
                v = (vf * torch.rsqrt(vf.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)).to(h.dtype).reshape(T, n_kv * D)
            qkv = torch.cat([q, k, v], dim=1).contiguous()
            qr, _ = ops.qk_norm_rope_append(qkv, nh, n_kv, D, w[f"{p}.attn.q_norm"], w[f"{p}.attn.k_norm"], cfg.rms_eps,
                                            cfg.norm_offset, cos_sin, rot, b.positions, slots, kv.k[il], kv.v[il], False)
        else:
            qn = ops.reference.head_rmsnorm(proj.view(T, nh, D), w[f"{p}.attn.q_norm"], cfg.rms_eps, cfg.norm_offset)
            qr = ops.reference.apply_rope(qn, cos_sin, b.positions, rot).to(h.dtype)
        o = ops.paged_attention(qr, kv.k[il], kv.v[il], table, b.ctx_lens, b.cu_q, b.max_q_len, cfg.attn_scale or 1.0,
                                window=cfg.sliding_window if swa else 0, decode_splits=b.decode_splits,
                                max_ctx=b.max_ctx or None)
        return ops.linear(o.reshape(T, -1), w[f"{p}.attn.o"])

    def _forward_gemma(self, b: StepBatch, kv: KvCache, want_logits: bool) -> StepOutput:
        """Forward pass of the Gemma-4 layer form (``src/model/gemma4.rs::gemma4_layers``): x = embed * scale; per
        layer attn_out = x + post_norm(attention(norm(x))); ffn = post_norm(dense FFN(norm(attn_out)) [MoE layers:
        post1(dense) + post2(routed experts over pre2(attn_out), routed by the scaled normed residual)]);
        x = (attn_out + ffn [+ per-layer embedding term]) * out_scale."""
        cfg, w, pc = self.cfg, self.w, self.pctx
        eps, off = cfg.rms_eps, cfg.norm_offset
        norm = lambda t, name: ops.rmsnorm(t, w[name], eps, off)[0]      # noqa: E731
        x0 = b.embeds if b.embeds is not None else self.embed(b.token_ids)
        dt = x0.dtype
        x = (x0.float() * cfg.embed_scale).to(dt)
        T = x.shape[0]
        ple = None
        if cfg.ple_dim:
            npl, L = cfg.ple_dim, cfg.n_layer
            rows = ops.embed(b.token_ids, w["ple_embd"]).float() * npl ** 0.5
            pr = (ops.linear(x, w["ple_model_proj"]).float() * cfg.hidden ** -0.5).view(T, L, npl)
            pr = pr * torch.rsqrt(pr.pow(2).mean(-1, keepdim=True) + eps) * (w["ple_proj_norm"].float() + off)
            ple = ((pr + rows.view(T, L, npl)) * 2 ** -0.5).to(dt)                          # [T, layer, npl]
        for il in range(cfg.n_layer):
            p = f"l{il}"
            a = self._gemma_attn(p, il, norm(x, f"{p}.attn_norm"), b, kv)
            attn_out = (norm(a, f"{p}.attn_post_norm").float() + x.float()).to(dt)
            n_ff = w[f"{p}.mlp.down"].shape[1]
            mlp = ops.linear(ops.gate_up_act(norm(attn_out, f"{p}.ffn_norm"), w[f"{p}.mlp.gate_up"], n_ff, cfg.ffn_act),
                             w[f"{p}.mlp.down"])
            if cfg.is_moe_layer(il):
                mlp = norm(mlp, f"{p}.ffn_post1_norm")
                af = attn_out.float()
                r = af * torch.rsqrt(af.pow(2).mean(-1, keepdim=True) + eps) * cfg.hidden ** -0.5
                r = (r * w[f"{p}.moe.router_scale"].float()).to(dt)
                routing = ops.router(r, w[f"{p}.moe.router"], cfg.top_k, "softmax", True, 1.0, None, 1, 1)
                moe_in = norm(attn_out, f"{p}.ffn_pre2_norm")
                y = ops.moe_experts(moe_in, routing.ids, routing.wts, w[f"{p}.moe.gate_up"], w[f"{p}.moe.down"],
                                    w[f"{p}.moe.down"].shape[2], cfg.ffn_act)
                mlp = (mlp.float() + norm(y, f"{p}.ffn_post2_norm").float()).to(dt)
            cur = (norm(mlp, f"{p}.ffn_post_norm").float() + attn_out.float()).to(dt)
            if ple is not None:
                t = torch.nn.functional.gelu(ops.linear(cur, w[f"{p}.ple.inp_gate"]).float(), approximate="tanh")
                t = ops.linear((t * ple[:, il].float()).to(dt), w[f"{p}.ple.proj"])
                cur = (cur.float() + norm(t, f"{p}.ple.post_norm").float()).to(dt)
            if cfg.layer_out_scale:
                cur = (cur.float() * w[f"{p}.out_scale"].float()).to(dt)
            x = cur
        rows = x if b.logit_rows is None else x.index_select(0, b.logit_rows)
        hidden, _ = ops.rmsnorm(rows, w["output_norm"], eps, off)
        out = StepOutput(hidden=hidden, last_hidden=x, captures={})
        if want_logits:
            out.logits = self.logits(hidden)
        pc.end_step()
        return out

    def _forward_blocks(self, b: StepBatch, kv: KvCache, st: Optional[StatePool], want_logits: bool) -> StepOutput:
        """One sub-layer per block (Nemotron-H as its checkpoints lay it out, ``src/model/nemotron_h.rs`` in the
        reference): x = x + sublayer(norm(x)), the sub-layer being a Mamba-2 mixer, attention without rotary
        embedding, a squared-ReLU FFN or the (latent) MoE. Runs on one rank from the framework's ops."""
        cfg, w, pc = self.cfg, self.w, self.pctx

        def whole(t):
            if isinstance(t, PendingLinear):
                return ops.linear(t.x, t.w)
            return t.materialize() if hasattr(t, "materialize") else t

        x = b.embeds if b.embeds is not None else self.embed(b.token_ids)
        for il in range(cfg.n_layer):
            p, kind = f"l{il}", cfg.layer_kinds[il]
            h = ops.rmsnorm(x, w[f"{p}.attn_norm"], cfg.rms_eps, cfg.norm_offset)[0]
            if kind in ("attn", "swa", "nope"):
                y = self._attn(p, il, h, b, kv, cfg.sliding_window if kind == "swa" else 0, rope=kind != "nope")
            elif kind == "mamba2":
                y = self._mamba2(p, il, h, b, st)
            elif kind in ("ffn", "moe"):
                y = self._ffn(p, kind == "moe", h, None)[0]
            else:
                raise ValueError(f"block form: unknown block kind {kind}")
            x = (x.float() + whole(y).float()).to(x.dtype)
        rows = x if b.logit_rows is None else x.index_select(0, b.logit_rows)
        hidden, _ = ops.rmsnorm(rows, w["output_norm"], cfg.rms_eps, cfg.norm_offset)
        out = StepOutput(hidden=hidden, last_hidden=x, captures={})
        if want_logits:
            out.logits = self.logits(hidden)
        pc.end_step()
        return out

    # ------------------------------------------------------------------ hyper-connections
    def _hc_pre(self, name: str, X):
        """Mixer in front of a sublayer (``ops.rs::cpu_hc_pre`` in the reference). X [T, hc, H] float32 streams ->
        (y [T, H]: the streams weighed into the sublayer's input, post [T, hc]: weight of the sublayer output in
        each new stream, comb [T, hc(dst), hc(src)]: Sinkhorn-normalised stream-to-stream mix)."""
        cfg, w = self.cfg, self.w
        T, hc, H = X.shape
        flat = X.reshape(T, hc * H)
        normed = flat * torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)
        mix = normed @ w[f"{name}.hc_f"].float().t()                                     # [T, (2 + hc) * hc]
        scale, base = w[f"{name}.hc_scale"].float(), w[f"{name}.hc_base"].float()
        eps = cfg.hc_eps
        pre = torch.sigmoid(mix[:, :hc] * scale[0] + base[:hc]) + eps
        post = torch.sigmoid(mix[:, hc:2 * hc] * scale[1] + base[hc:2 * hc]) * 2.0
        # comb[t, s, d] laid out source-major like the reference's buffer (d fastest)
        cm = (mix[:, 2 * hc:] * scale[2] + base[2 * hc:]).view(T, hc, hc)
        cm = torch.softmax(cm, dim=2) + eps                       # over destinations, per source
        cm = cm / (cm.sum(1, keepdim=True) + eps)                 # each destination over the sources
        for _ in range(1, cfg.hc_iters):
            cm = cm / (cm.sum(2, keepdim=True) + eps)             # each source over the destinations
            cm = cm / (cm.sum(1, keepdim=True) + eps)
        y = (X * pre.unsqueeze(-1)).sum(1)
        return y, post, cm.transpose(1, 2).contiguous()

    def _hcg_mix(self, name: str, X, inject: bool):
        """Gated mixer (qwen4exp; ``src/model/qwen4.rs::hc_mix`` in the reference): every stream is RMS-normed with
        a weight of its own; a low-rank gate ``up(silu(down(xn) / hc))`` gives a sigmoid weight per stream and
        channel; the block input is the mean of the gated streams. With ``inject`` also the per-stream logits of
        the weights the block output re-enters the streams with."""
        cfg, w = self.cfg, self.w
        T, hc, H = X.shape
        xn = X * torch.rsqrt(X.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * w[f"{name}.hcg_norm"].float()
        flat = xn.reshape(T, hc * H)
        inj = flat @ w[f"{name}.hcg_inject"].float().t() if inject else None
        lo = torch.nn.functional.silu((flat @ w[f"{name}.hcg_down"].float().t()) / hc)
        gate = (lo @ w[f"{name}.hcg_up"].float().t()).view(T, hc, H)
        return (xn * torch.sigmoid(gate)).sum(1) / hc, inj

    @staticmethod
    def _hcg_combine(out, X, inj):
        """Stream h += out * 2 sigmoid(inject[h] / hc)."""
        return X + out.float().unsqueeze(1) * (2.0 * torch.sigmoid(inj / X.shape[1])).unsqueeze(-1)

    @staticmethod
    def _hc_post(out, X, post, comb):
        """New stream d = out * post[d] + sum_s X[s] * comb[d, s]."""
        return out.float().unsqueeze(1) * post.unsqueeze(-1) + torch.einsum("tds,tsh->tdh", comb, X)

    def _forward_hc(self, b: StepBatch, kv: KvCache, st: Optional[StatePool], want_logits: bool) -> StepOutput:
        """Forward pass of a model whose residual is several streams (hyper-connections). Every sublayer reads
        the streams through its own mixer and its output re-enters every stream with per-token weights
        (``src/model/glm5next.rs:994-1036`` in the reference); the head reads the streams' mean."""
        cfg, w, pc = self.cfg, self.w, self.pctx
        hc = cfg.hyper_streams
        x0 = b.embeds if b.embeds is not None else self.embed(b.token_ids)
        dt = x0.dtype
        X = x0.float().unsqueeze(1).expand(-1, hc, -1).contiguous()
        gated = cfg.hyper_mode == "gated"
        for il in range(cfg.n_layer):
            p, kind = f"l{il}", cfg.layer_kinds[il]
            if gated:
                y, inj = self._hcg_mix(f"{p}.hca", X, True)
                h = y.to(dt)
            else:
                y, post, comb = self._hc_pre(f"{p}.hca", X)
                h, _ = ops.rmsnorm(y.to(dt), w[f"{p}.attn_norm"], cfg.rms_eps, cfg.norm_offset)
            if kind in ("attn", "swa", "nope"):
                a = self._attn(p, il, h, b, kv, cfg.sliding_window if kind == "swa" else 0, rope=kind != "nope")
            elif kind == "gdn":
                a = self._gdn(p, il, h, b, st)
            elif kind == "mla":
                a = self._mla(p, il, h, b, kv)
            elif kind == "kda":
                a = self._kda(p, il, h, b, st)
            elif kind == "mamba2":
                a = self._mamba2(p, il, h, b, st)
            else:
                raise ValueError(kind)
            a = pc.full_hidden(a, None)
            if gated:
                X = self._hcg_combine(a, X, inj)
                y, inj = self._hcg_mix(f"{p}.hcf", X, True)
                h = y.to(dt)
            else:
                X = self._hc_post(a, X, post, comb)
                y, post, comb = self._hc_pre(f"{p}.hcf", X)
                h, _ = ops.rmsnorm(y.to(dt), w[f"{p}.ffn_norm"], cfg.rms_eps, cfg.norm_offset)
            f, _, _ = self._ffn(p, cfg.is_moe_layer(il), h, None)
            f = pc.full_hidden(f, None)
            X = self._hcg_combine(f, X, inj) if gated else self._hc_post(f, X, post, comb)
        last = X.mean(1).to(dt)
        if gated:
            Xr = X if b.logit_rows is None else X.index_select(0, b.logit_rows)
            hidden = self._hcg_mix("out_hc", Xr, False)[0].to(dt)         # the last mixer is the output norm
        else:
            rows = last if b.logit_rows is None else last.index_select(0, b.logit_rows)
            hidden, _ = ops.rmsnorm(rows, w["output_norm"], cfg.rms_eps, cfg.norm_offset)
        out = StepOutput(hidden=hidden, last_hidden=last, captures={})
        if want_logits:
            out.logits = self.logits(hidden)
        pc.end_step()
        return out

    def _mamba2(self, p: str, il: int, x, b: StepBatch, st: StatePool):
        """Mamba-2 (SSD) layer: on a GPU the recurrence, the D skip and the silu(z) gate are one kernel with the state
        of a (sequence, head) in registers (``csrc/mamba2.cu``); the CPU form is the token-serial reference."""
        cfg, w = self.cfg, self.w
        nh, hd, ng, ds = cfg.ssm_heads, cfg.ssm_head_dim, cfg.ssm_groups, cfg.ssm_state
        di = nh * hd
        T = x.shape[0]
        proj = ops.linear(x, w[f"{p}.ssm.in"])
        z, xbc, dt = proj[:, :di], proj[:, di:2 * di + 2 * ng * ds], proj[:, 2 * di + 2 * ng * ds:]
        xbc = ops.causal_conv1d_silu(xbc.contiguous(), w[f"{p}.ssm.conv_w"], w[f"{p}.ssm.conv_b"], st.conv[il], b.cu_q,
                                     b.state_slots, write_state=b.write_state)
        if x.is_cuda and ops.sm100.mamba2_scan_ok(nh, hd, ng, ds) and x.dtype == torch.bfloat16:
            yz = ops.sm100.mamba2_scan(xbc, dt, z, w[f"{p}.ssm.A"], w[f"{p}.ssm.D"], w[f"{p}.ssm.dt_bias"], st.ssm[il],
                                       b.cu_q, b.state_slots, nh, hd, ng, ds, write_state=b.write_state)
            if ng > 1:
                # the gated norm works per group of channels: unit-weight norm over each group, then the weights
                g = ops.rmsnorm(yz.view(T * ng, di // ng), self._ones(di // ng, yz), cfg.rms_eps, 0.0)[0]
                yn = (g.view(T, di).float() * w[f"{p}.ssm.norm"].float()).to(yz.dtype)
            else:
                yn, _ = ops.rmsnorm(yz, w[f"{p}.ssm.norm"], cfg.rms_eps, 0.0)
            return ops.linear(yn, w[f"{p}.ssm.out"])
        xs = xbc[:, :di].float().view(T, nh, hd)
        Bm = xbc[:, di:di + ng * ds].float().view(T, ng, ds)
        Cm = xbc[:, di + ng * ds:].float().view(T, ng, ds)
        dtv = F.softplus(dt.float() + w[f"{p}.ssm.dt_bias"])
        A = w[f"{p}.ssm.A"].float()
        Dp = w[f"{p}.ssm.D"].float()
        y = torch.empty(T, nh, hd, device=x.device, dtype=torch.float32)
        cu = b.cu_q_host if b.cu_q_host is not None else b.cu_q.tolist()
        slots = b.state_slots.tolist()
        hg = nh // ng
        for i in range(b.n_seqs):
            S = st.ssm[il][slots[i]].clone()
            for t in range(cu[i], cu[i + 1]):
                dA = torch.exp(dtv[t] * A)[:, None, None]
                Bt = Bm[t].repeat_interleave(hg, dim=0)
                Ct = Cm[t].repeat_interleave(hg, dim=0)
                S = S * dA + (dtv[t][:, None] * xs[t])[:, :, None] * Bt[:, None, :]
                y[t] = torch.einsum("hds,hs->hd", S, Ct) + Dp[:, None] * xs[t]
            if b.write_state:
                st.ssm[il][slots[i]] = S
        yz = (y.view(T, di) * F.silu(z.float())).view(T, ng, di // ng)       # the gated norm works per group
        yn = (yz * torch.rsqrt(yz.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)).view(T, di) * w[f"{p}.ssm.norm"].float()
        return ops.linear(yn.to(x.dtype), w[f"{p}.ssm.out"])

    def _ones(self, n: int, like) -> torch.Tensor:
        key = (n, like.device)
        cache = self.__dict__.setdefault("_ones_cache", {})
        if key not in cache:
            cache[key] = torch.ones(n, device=like.device, dtype=torch.float32)      # norm weights are float32
        return cache[key]

    def _route(self, p: str, x, norm=None):
        cfg, w, pc = self.cfg, self.w, self.pctx
        e_lo, e_hi = pc.expert_range(cfg.n_expert)
        kw = {}
        if x.is_cuda:
            stacked = w.get(f"{p}.moe.gate_up_s")
            if stacked is not None:     # the shared expert rides in the grouped GEMMs of decode-sized steps
                kw = dict(shared_slot=True, sh_gate=w.get(f"{p}.moe.sh_gate") if cfg.shared_gate else None)
            if isinstance(stacked if stacked is not None else w.get(f"{p}.moe.gate_up"), ops.sm100.Nv4Weight):
                kw["slot_stride"] = 128
        return ops.router(x, w[f"{p}.moe.router"], cfg.top_k, cfg.router_mode, cfg.norm_topk,
                          cfg.route_scale, w.get(f"{p}.moe.router_bias"), cfg.n_group, cfg.topk_group,
                          e_lo=e_lo, n_local=e_hi - e_lo, norm=norm, **kw)

    def _ffn(self, p: str, il_moe: bool, x, residual, next_norm=None, routing=None):
        """Returns (out, fused, normed). ``fused``: the residual is already added (TP == 1). ``normed``: the
        next layer's input norm of ``out`` when ``next_norm`` was given and the MoE combine could carry it.
        ``routing``: the router's result when the caller already ran it (with the FFN norm inside)."""
        cfg, w, pc = self.cfg, self.w, self.pctx
        fuse_res = residual is not None and pc.tp == 1
        if il_moe:
            if routing is None:
                routing = self._route(p, x)
            ids, wts = routing
            shared = gate = None
            folded = bool(getattr(routing, "shared_slot", False))
            if cfg.shared_ff > 0 and not folded and w.get(f"{p}.moe.sh_down") is not None:
                fs = w[f"{p}.moe.sh_down"].shape[1]
                xs = x
                if (x.is_cuda and isinstance(w[f"{p}.moe.sh_gate_up"], ops.sm100.Fp8Weight)
                        and isinstance(w.get(f"{p}.moe.gate_up"), ops.sm100.Fp8Weight) and x.shape[0] <= 64):
                    # FP8 shared and routed experts read the same rows: encode them once
                    xs = ops.sm100.Fp8Act.of(x)
                    if isinstance(routing, ops.sm100.Routing):
                        routing.xq = xs
                hs = ops.gate_up_act(xs, w[f"{p}.moe.sh_gate_up"], fs, cfg.ffn_act)
                shared = ops.linear(hs, w[f"{p}.moe.sh_down"])
                if cfg.shared_gate:
                    gate = ops.linear(x, w[f"{p}.moe.sh_gate"], out_dtype=torch.float32).reshape(-1).contiguous()
            e_lo, _ = pc.expert_range(cfg.n_expert)
            cache = self.expert_cache.get(p)
            if cache is not None:
                # offloaded experts: make this step's experts resident, then route by slot number
                ids = cache.prepare(ids)
                w_gu, w_dn = cache.weights()
                e_lo = 0
                routing = None
            elif folded:
                w_gu, w_dn = w[f"{p}.moe.gate_up_s"], w[f"{p}.moe.down_s"]
            else:
                w_gu, w_dn = w[f"{p}.moe.gate_up"], w[f"{p}.moe.down"]
            n_ff = w_dn.shape[2]
            if cfg.moe_latent:
                # latent MoE: the routed experts run between a down and an up projection; the shared expert (full
                # width) joins after the up projection. Every piece is linear in the rank-partial sums.
                xl = ops.linear(x, w[f"{p}.moe.lat_down"])
                y = pc.moe(xl, ids, wts, w_gu, w_dn, n_ff, cfg.ffn_act, e_lo, None, None, None,
                           routing=routing if x.is_cuda else None)
                if hasattr(y, "materialize"):
                    y = y.materialize()
                out = ops.linear(y, w[f"{p}.moe.lat_up"])
                if shared is not None:
                    sh = shared.float() * (torch.sigmoid(gate.float())[:, None] if gate is not None else 1.0)
                    out = (out.float() + sh).to(out.dtype)
                return out, False, None
            if fuse_res and next_norm is not None:
                out, normed = pc.moe(x, ids, wts, w_gu, w_dn, n_ff, cfg.ffn_act, e_lo, shared, gate, residual,
                                     norm=(next_norm, cfg.rms_eps, cfg.norm_offset), routing=routing)
                return out, True, normed
            return pc.moe(x, ids, wts, w_gu, w_dn, n_ff, cfg.ffn_act, e_lo, shared, gate,
                          residual if fuse_res else None, routing=routing), fuse_res, None
        n_ff = w[f"{p}.mlp.down"].shape[1]
        h = ops.gate_up_act(x, w[f"{p}.mlp.gate_up"], n_ff, cfg.ffn_act)
        if fuse_res:
            return ops.linear(h, w[f"{p}.mlp.down"], residual=residual), True, None
        return pc.defer_linear(h, w[f"{p}.mlp.down"]), False, None

    def _layer(self, p: str, il: int, kind: str, moe: bool, x, resid, b, kv, st, pre_normed=None, next_norm=None):
        """x is the (possibly rank-partial) output of the previous sub-layer, resid the residual stream.
        ``pre_normed``: this layer's input norm, already computed by the previous layer's combine.
        Returns (cur, res, normed_for_next_layer or None)."""
        cfg, w, pc = self.cfg, self.w, self.pctx
        if pre_normed is not None:
            h = pre_normed
        else:
            h, resid = pc.reduce_norm(x, resid, w[f"{p}.attn_norm"], cfg.rms_eps, cfg.norm_offset)
        if kind in ("attn", "swa", "nope"):
            a = self._attn(p, il, h, b, kv, cfg.sliding_window if kind == "swa" else 0, rope=kind != "nope")
        elif kind == "gdn":
            a = self._gdn(p, il, h, b, st)
        elif kind == "mla":
            a = self._mla(p, il, h, b, kv)
        elif kind == "mamba2":
            a = self._mamba2(p, il, h, b, st)
        elif kind == "kda":
            a = self._kda(p, il, h, b, st)
        else:
            raise ValueError(kind)
        routing = None
        nv4_decode = False
        a_rows = a.x if isinstance(a, PendingLinear) else a
        if moe and resid is not None and a_rows.is_cuda and a_rows.shape[0] <= 64 and self.expert_cache.get(p) is None \
                and (isinstance(a, PendingLinear) or pc.world > 1):
            wg = w.get(f"{p}.moe.gate_up_s")
            nv4_decode = isinstance(wg if wg is not None else w.get(f"{p}.moe.gate_up"), ops.sm100.Nv4Weight)
        if nv4_decode and pc.world > 1:
            # several ranks: the reduction launch adds the residual, applies the FFN norm and encodes the rows
            h, resid, xq = pc.reduce_norm_quant(a, resid, w[f"{p}.ffn_norm"], cfg.rms_eps, cfg.norm_offset)
            routing = self._route(p, h)
            routing.xq = xq
        elif nv4_decode:
            # decode-sized step on NVFP4 experts: one launch adds the residual, applies the FFN norm and encodes the
            # normalised rows for the expert GEMMs; the router reads the bf16 copy
            att = ops.linear(a.x, a.w)
            xq = ops.sm100.nv4_quant_act(att, norm=(w[f"{p}.ffn_norm"], cfg.rms_eps, cfg.norm_offset), residual=resid,
                                         want_normed=True, key="ffn_in")
            resid, h = xq.summed, xq.normed
            routing = self._route(p, h)
            routing.xq = xq
        elif moe and pc.world == 1 and isinstance(a, PendingLinear) and resid is not None and ops.sm100.TUNE["route_norm"]:
            # single rank: the projection's epilogue adds the residual and the routing launch applies the FFN norm
            resid = ops.linear(a.x, a.w, residual=resid)
            routing = self._route(p, resid, norm=(w[f"{p}.ffn_norm"], cfg.rms_eps, cfg.norm_offset))
            h = routing.x_normed
        else:
            h, resid = pc.reduce_norm(a, resid, w[f"{p}.ffn_norm"], cfg.rms_eps, cfg.norm_offset)
        f, fused, normed = self._ffn(p, moe, h, resid, next_norm, routing)
        if fused:
            return None, f, normed  # residual already folded in: f is the new residual stream
        return f, resid, None

    # ------------------------------------------------------------------ forward
    def embed(self, token_ids):
        return ops.embed(token_ids, self.w["tok_embd"])

    def embed_dtype(self):
        """dtype of the rows ``embed`` gives (image rows are cast to it)."""
        dt = getattr(self, "_embed_dtype", None)
        if dt is None:
            dev = self.cos_sin.device
            dt = self.embed(torch.zeros(1, dtype=torch.int32, device=dev)).dtype
            self._embed_dtype = dt
        return dt

    def _forward_pipe(self, b: StepBatch, kv: KvCache, st: Optional[StatePool], want_logits: bool) -> StepOutput:
        """Pipeline-parallel forward: this rank's layers over the step's micro-chunks. The receive of micro-chunk
        c+1 is posted before c is computed and sends are asynchronous, so neighbouring stages overlap."""
        cfg, w, pc, pipe = self.cfg, self.w, self.pctx, self.pipe
        chunks = pipe.plan(b)
        sizes = [int(c.token_ids.shape[0]) if c.embeds is None else int(c.embeds.shape[0]) for c in chunks]
        recvs, sends, outs = {}, [], []
        if not pipe.first:
            recvs[0] = pipe.irecv(sizes[0], cfg.hidden, self.dtype, self.device)
        for i, c in enumerate(chunks):
            if pipe.first:
                cur, res = (c.embeds if c.embeds is not None else self.embed(c.token_ids)), None
            else:
                buf, work = recvs.pop(i)
                if i + 1 < len(chunks):
                    recvs[i + 1] = pipe.irecv(sizes[i + 1], cfg.hidden, self.dtype, self.device)
                work.wait()
                cur, res = None, buf
            normed = None
            for il in range(pipe.lo, pipe.hi):
                nxt = w[f"l{il + 1}.attn_norm"] if il + 1 < pipe.hi else None
                cur, res, normed = self._layer(f"l{il}", il, cfg.layer_kinds[il], cfg.is_moe_layer(il), cur, res, c, kv,
                                               st, normed, nxt)
            hid = pc.full_hidden(cur, res)
            if pipe.last:
                outs.append(hid)
            else:
                sends.append((hid, pipe.isend(hid)))
        for _, work in sends:
            work.wait()
        T = sum(sizes)
        R = T if b.logit_rows is None else int(b.logit_rows.shape[0])
        if pipe.last:
            last = outs[0] if len(outs) == 1 else torch.cat(outs, 0)
            rows = last if b.logit_rows is None else last.index_select(0, b.logit_rows)
            hidden, _ = ops.rmsnorm(rows, w["output_norm"], cfg.rms_eps, cfg.norm_offset)
            logits = self.logits(hidden) if want_logits else None
        else:
            last = None
            hidden = torch.empty(R, cfg.hidden, dtype=self.dtype, device=self.device)
            logits = torch.empty(R, cfg.vocab, dtype=torch.float32, device=self.device) if want_logits else None
        pipe.broadcast_from_last(hidden)
        if want_logits:
            pipe.broadcast_from_last(logits)
        pc.end_step()
        return StepOutput(hidden=hidden, logits=logits, last_hidden=last, captures={})

    def forward(self, b: StepBatch, kv: KvCache, st: Optional[StatePool], want_logits: bool = True) -> StepOutput:
        if self.pipe is not None:
            return self._forward_pipe(b, kv, st, want_logits)
        if self.cfg.hyper_streams > 1:
            return self._forward_hc(b, kv, st, want_logits)
        if self.cfg.sandwich_norm:
            return self._forward_gemma(b, kv, want_logits)
        if self.cfg.block_form:
            return self._forward_blocks(b, kv, st, want_logits)
        cfg, w, pc = self.cfg, self.w, self.pctx
        x = b.embeds if b.embeds is not None else self.embed(b.token_ids)
        resid = None
        x_partial = False
        captures: Dict[int, torch.Tensor] = {}
        cur, res = x, None
        # The stream is carried as (cur, res): hidden = cur (+ res). After the embedding res is None.
        normed = None
        for il in range(cfg.n_layer):
            nxt = w[f"l{il + 1}.attn_norm"] if il + 1 < cfg.n_layer else None
            cur, res, normed = self._layer(f"l{il}", il, cfg.layer_kinds[il], cfg.is_moe_layer(il), cur, res, b, kv,
                                           st, normed, nxt)
            if b.deepstack is not None and il < len(b.deepstack):
                # image tokens: the tower's extra rows for this depth join the residual stream
                full = pc.full_hidden(cur, res)
                full.index_add_(0, b.deepstack_rows, b.deepstack[il].to(full.dtype))
                cur, res, normed = None, full, None
            if b.capture_layers and il in b.capture_layers:
                captures[il] = pc.full_hidden(cur, res)
        last = pc.full_hidden(cur, res)
        rows = last if b.logit_rows is None else last.index_select(0, b.logit_rows)
        hidden, _ = ops.rmsnorm(rows, w["output_norm"], cfg.rms_eps, cfg.norm_offset)
        out = StepOutput(hidden=hidden, last_hidden=last, captures=captures)
        if want_logits:
            out.logits = self.logits(hidden)
        pc.end_step()
        _ = (resid, x_partial)
        return out

    def mrope_table(self, pos3: torch.Tensor) -> torch.Tensor:
        """[3, T] positions on the (temporal, row, column) axes -> [T, rot] cos | sin rows: frequency i turns with
        the axis the model's section layout gives it (``vision.media.mrope_axis_of_freq``), so each row is a gather
        from the ordinary table at that axis' position."""
        from ..vision.media import mrope_axis_of_freq
        half = self.cos_sin.shape[1] // 2
        ax = getattr(self, "_mrope_axis", None)
        if ax is None:
            ax = mrope_axis_of_freq(half, self.cfg.mrope_sections, self.cfg.mrope_interleaved).to(self.cos_sin.device)
            self._mrope_axis = ax
        pos3 = pos3.to(self.cos_sin.device)
        rows = pos3[ax].t()                                        # [T, half]: the position frequency i reads
        cols = torch.arange(half, device=rows.device)
        return torch.cat([self.cos_sin[rows, cols], self.cos_sin[rows, cols + half]], dim=1).contiguous()

    def split_head(self) -> bool:
        """Several ranks with the fused communicator: every rank keeps only its slice of the LM head's vocabulary
        rows (the reference's ``src/model/core/head_split.rs``), so a step reads 1 / world of the head. Greedy
        steps exchange (best value, token id) pairs (``greedy_picks``); callers that need the logits themselves get
        them gathered (``logits``). Returns whether the head was split."""
        pc = self.pctx
        V = self.lm_head.shape[0]
        if (self.head_split is not None or pc.world <= 1 or pc.comm != "fused" or pc.symm is None or V % pc.world
                or not isinstance(self.lm_head, torch.Tensor) or not self.lm_head.is_cuda):
            return False
        n = V // pc.world
        self.head_split = (pc.rank * n, n)
        self.lm_head = self.lm_head[pc.rank * n:(pc.rank + 1) * n].contiguous()
        if "output" in self.w:
            self.w["output"] = self.lm_head         # the full copy is released
        return True

    def _local_logits(self, hidden):
        lg = ops.linear(hidden, self.lm_head, out_dtype=torch.float32)
        if self.cfg.logit_scale != 1.0:
            lg = lg * self.cfg.logit_scale
        if self.cfg.logit_softcap > 0:
            lg = torch.tanh(lg / self.cfg.logit_softcap) * self.cfg.logit_softcap
        return lg

    def gather_logits(self, local):
        """[rows, vocab / world] of every rank -> [rows, vocab] on every rank."""
        import torch.distributed as dist
        pc = self.pctx
        R, n = local.shape
        parts = torch.empty(pc.world, R, n, dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(parts, local.contiguous(), group=pc.group)
        return parts.permute(1, 0, 2).reshape(R, pc.world * n)

    def greedy_picks(self, hidden, out):
        """Arg-max token of every row of ``hidden`` (already normalised) into ``out`` (int32). With a split head only
        (value, token id) pairs cross the ranks. Returns this rank's logits (its vocabulary slice when split)."""
        lg = self._local_logits(hidden)
        if self.head_split is None:
            ops.sm100.argmax(lg, out=out)
            return lg
        R = lg.shape[0]
        ws = ops.sm100.Workspace.get(lg.device)
        val = ws.buf("head_val", (R,), torch.float32)
        idx = ws.buf("head_idx", (R,), torch.int32)
        ops.sm100.argmax(lg, out=idx, out_val=val)
        self.pctx.symm.argmax_exchange(val, idx, self.head_split[0], out)
        return lg

    def logits(self, hidden):
        lg = self._local_logits(hidden)
        return self.gather_logits(lg) if self.head_split is not None else lg

    def commit_replay(self, b: StepBatch, st: StatePool, commits):
        """After a verify step (state not advanced): replays the kept tokens of each sequence through the
        conv window and the delta rule so the state equals sequential decoding of exactly those tokens.
        ``commits`` = [(sequence index in the batch, kept tokens)]. The reference does the same with a
        replay pool of (q, k, v, g, beta) rows (``src/model/core/spec.rs:1-12``, ``Executor::commit``)."""
        if not b.replay:
            return
        cfg, w = self.cfg, self.w
        cu = b.cu_q_host if b.cu_q_host is not None else b.cu_q.tolist()
        rows, new_cu, seqs = [], [0], []
        for bi, kept in commits:
            if kept <= 0:
                continue
            rows.extend(range(cu[bi], cu[bi] + kept))
            new_cu.append(new_cu[-1] + kept)
            seqs.append(bi)
        if not rows:
            return
        dev = b.token_ids.device
        idx = torch.tensor(rows, dtype=torch.long, device=dev)
        cu_t = torch.tensor(new_cu, dtype=torch.int32, device=dev)
        slots = b.state_slots[torch.tensor(seqs, dtype=torch.long, device=dev)].contiguous()
        for il, (mixed, g, beta) in b.replay.items():
            p = f"l{il}"
            conv = ops.causal_conv1d_silu(mixed.index_select(0, idx).contiguous(), w[f"{p}.gdn.conv_w"], None,
                                          st.conv[il], cu_t, slots, write_state=True)
            ops.gdn_recurrent(conv, g.index_select(0, idx).contiguous(), beta.index_select(0, idx).contiguous(),
                              st.ssm[il], cu_t, slots, self.gdn_k_l, self.gdn_v_l, cfg.gdn_k_dim, cfg.gdn_v_dim,
                              cfg.gdn_tiled_heads, cfg.gdn_k_dim ** -0.5, 1e-6, write_state=True)

    # ------------------------------------------------------------------ MTP head
    def mtp_forward(self, j: int, b: StepBatch, prev_hidden, kv: KvCache, st: Optional[StatePool]) -> StepOutput:
        """Draft head j: tokens b.token_ids at positions b.positions with the target's (or the head's own)
        hidden row of the previous position in ``prev_hidden`` [T, H]."""
        cfg, w, pc = self.cfg, self.w, self.pctx
        p = f"mtp{j}"
        e, _ = ops.rmsnorm(self.embed(b.token_ids), w[f"{p}.enorm"], cfg.rms_eps, cfg.norm_offset)
        hprev, _ = ops.rmsnorm(prev_hidden, w[f"{p}.hnorm"], cfg.rms_eps, cfg.norm_offset)
        x = ops.linear(torch.cat([e, hprev], dim=-1), w[f"{p}.eh_proj"])
        kind = "mla" if cfg.kv_lora > 0 else "attn"
        cur, res, _ = self._layer(f"{p}.l", cfg.n_layer + j, kind, cfg.n_expert > 0, x, None, b, kv, st)
        last = pc.full_hidden(cur, res)
        rows = last if b.logit_rows is None else last.index_select(0, b.logit_rows)
        hidden, _ = ops.rmsnorm(rows, w[f"{p}.shared_head_norm"], cfg.rms_eps, cfg.norm_offset)
        return StepOutput(hidden=hidden, logits=self.logits(hidden), last_hidden=last)
