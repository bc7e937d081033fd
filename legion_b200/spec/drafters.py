"""Drafters. Model-free ones implement ``propose(seq, k)``; model drafters implement ``on_step`` (see every
target step: keep their own KV in step with the sequence) and ``draft_batch`` (chain k drafts after a step).

Reference: ``src/spec/ngram.rs``, ``suffix.rs``, ``draft.rs``, ``eagle3.rs`` (+ ``eagle3/config.rs:22-62``),
``dflash.rs``, MTP in the executor (``src/model/core/exec.rs:1864``, ``src/model/qwen35/mtp.rs:1-14``).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..config import ModelConfig
from ..models.decoder import Decoder, KvCache, StatePool


class Drafter:
    model_free = True
    needs_hidden = False
    capture_layers: Optional[List[int]] = None

    def propose(self, seq, k: int) -> List[int]:
        return []

    def on_step(self, items, batch, out):
        pass

    def draft_batch(self, seqs, k: int):
        pass

    def release(self, seq):
        pass


class NgramDrafter(Drafter):
    """Prompt lookup: find the most recent earlier occurrence of the sequence's last n tokens (longest n
    first) and propose what followed it."""

    def __init__(self, n_min: int = 2, n_max: int = 4):
        self.n_min, self.n_max = n_min, n_max

    def propose(self, seq, k):
        t = seq.tokens
        L = len(t)
        for n in range(min(self.n_max, L - 1), self.n_min - 1, -1):
            tail = t[L - n:]
            for i in range(L - n - 1, -1, -1):
                if t[i:i + n] == tail:
                    return list(t[i + n:i + n + k])
        return []


class SuffixDrafter(Drafter):
    """Suffix index over everything seen: the running sequence plus finished replies of earlier requests
    (a cross-request cache). Proposes the continuation of the longest suffix that occurred before."""

    def __init__(self, max_suffix: int = 8, cache_tokens: int = 1 << 18):
        self.max_suffix, self.cache_tokens = max_suffix, cache_tokens
        self.index: Dict[tuple, tuple] = {}      # n-gram -> (corpus id, position after it)
        self.corpus: Dict[int, List[int]] = {}
        self._next_id = 0
        self._size = 0

    def _add(self, toks: List[int]):
        cid = self._next_id
        self._next_id += 1
        self.corpus[cid] = list(toks)
        self._size += len(toks)
        for n in range(2, self.max_suffix + 1):
            for i in range(0, len(toks) - n):
                self.index[tuple(toks[i:i + n])] = (cid, i + n)
        while self._size > self.cache_tokens and self.corpus:
            old = min(self.corpus)
            self._size -= len(self.corpus.pop(old))

    def propose(self, seq, k):
        t = seq.tokens
        own = NgramDrafter(2, self.max_suffix).propose(seq, k)
        if own:
            return own
        for n in range(min(self.max_suffix, len(t)), 1, -1):
            hit = self.index.get(tuple(t[-n:]))
            if hit and hit[0] in self.corpus:
                c = self.corpus[hit[0]]
                return c[hit[1]:hit[1] + k]
        return []

    def release(self, seq):
        if seq.n_out > 0:
            self._add(seq.tokens)


class _ModelDrafter(Drafter):
    model_free = False
    needs_hidden = True

    def __init__(self, engine):
        self.eng = engine
        self.prev: Dict[int, torch.Tensor] = {}    # id(seq) -> hidden row paired with the next token

    def release(self, seq):
        self.prev.pop(id(seq), None)

    def _zeros(self, H):
        return torch.zeros(H, device=self.eng.device, dtype=self.eng.model.dtype)


class MtpDrafter(_ModelDrafter):
    """The model's own MTP head: input row for position p = eh_proj([norm(embed(tok_p)); norm(h_{p-1})]) where
    h is the target's residual stream (or, when chaining, the head's own output). The head's KV lives in the
    target's blocks (an extra layer of the KV cache), so prefix-cache hits cover it too."""

    def __init__(self, engine):
        super().__init__(engine)
        assert engine.mcfg.mtp_layers > 0, "--spec mtp needs a model with an MTP head"

    def on_step(self, items, b, out):
        eng = self.eng
        H = eng.mcfg.hidden
        cu = b.cu_q_host
        fill, prevs = [], []
        for s, p0, fed, kept, bi in items:
            if kept <= 0:
                continue
            rows = out.last_hidden[cu[bi]:cu[bi] + kept]
            first = self.prev.get(id(s))
            if first is None:
                first = self._zeros(H)
            prevs.append(torch.cat([first[None], rows[:kept - 1]], dim=0))
            fill.append((s, p0, fed[:kept]))
            self.prev[id(s)] = rows[kept - 1].clone()
        if fill:
            mb = eng.build_batch_explicit(fill)
            eng.model.mtp_forward(0, mb, torch.cat(prevs, dim=0), eng.kv, eng.states)

    def draft_batch(self, seqs, k):
        eng = self.eng
        live = [s for s in seqs if id(s) in self.prev]
        for s in live:
            s.drafts = []
        hidden = {id(s): self.prev[id(s)] for s in live}
        for j in range(k):
            items, prevs = [], []
            for s in live:
                pos = len(s.tokens) - 1 + j
                if pos + 2 >= eng.cfg.ctx_size or pos >= s.table.capacity(eng.pool):
                    continue
                tok = s.tokens[-1] if j == 0 else s.drafts[j - 1]
                items.append((s, pos, [tok]))
                prevs.append(hidden[id(s)][None])
            if not items:
                break
            mb = eng.build_batch_explicit(items)
            o = eng.model.mtp_forward(0, mb, torch.cat(prevs, dim=0), eng.kv, eng.states)
            picks = ops.argmax(o.logits).tolist()
            for (s, _, _), t, row in zip(items, picks, o.last_hidden):
                s.drafts.append(int(t))
                hidden[id(s)] = row


class MtpNgramDrafter(MtpDrafter):
    """MTP head with a prompt-lookup shortcut: a sequence whose last tokens occurred before takes the tokens that
    followed them as its drafts (no head launches for it in this step); the others chain the MTP head, and an MTP
    chain is extended by looking its own drafts up the same way. The head still sees every target step, so its KV
    stays in step either way. Reference: ``src/engine/lm/mtp_ngram.rs``."""

    def __init__(self, engine, n_min: int = 2, n_max: int = 4, extend: int = 2):
        super().__init__(engine)
        self.ngram = NgramDrafter(n_min, n_max)
        self.extend = extend
        self.stats = {"ngram_hits": 0, "mtp_chains": 0, "extended": 0}

    def draft_batch(self, seqs, k):
        chain = []
        for s in seqs:
            if id(s) not in self.prev:
                continue
            got = self.ngram.propose(s, k)
            if len(got) >= min(2, k):
                s.drafts = got
                self.stats["ngram_hits"] += 1
            else:
                chain.append(s)
        if chain:
            self.stats["mtp_chains"] += len(chain)
            super().draft_batch(chain, k)
            for s in chain:
                if len(s.drafts) == k and self.extend > 0:
                    class _View:        # the sequence continued by its own drafts
                        tokens = s.tokens + s.drafts
                    more = self.ngram.propose(_View, self.extend)
                    room = self.eng.cfg.ctx_size - len(s.tokens) - len(s.drafts) - 2
                    if more and room > 0:
                        s.drafts = s.drafts + more[:room]
                        self.stats["extended"] += 1


class DraftModelDrafter(_ModelDrafter):
    """A separate (smaller) model with the target's vocabulary. It sees every token the target sees (own KV in
    the same block ids) and then runs k greedy steps ahead."""

    def __init__(self, engine, draft: Optional[Decoder] = None):
        super().__init__(engine)
        self.draft = draft if draft is not None else engine.model
        if self.draft.cfg.vocab != engine.mcfg.vocab:
            raise ValueError("the draft model must use the target's vocabulary")
        self.kv = KvCache(self.draft.cfg, engine.pool.total, engine.cfg.block_size, engine.device, self.draft.dtype,
                          kv_heads_local=self.draft.n_kv_l)
        self.hybrid = bool(self.draft.cfg.recurrent_layers())
        self.states = StatePool(self.draft.cfg, engine.cfg.max_seqs + 1, engine.device) if self.hybrid else None
        self.state_saved = StatePool(self.draft.cfg, engine.cfg.max_seqs + 1, engine.device) if self.hybrid else None
        self.filled: Dict[int, int] = {}

    def on_step(self, items, b, out):
        eng = self.eng
        fill = []
        for s, p0, fed, kept, bi in items:
            if kept <= 0:
                continue
            done = self.filled.get(id(s), 0)
            if done < p0:       # resumed from the prefix cache: the draft model has to read the prefix itself
                fill.append((s, done, s.tokens[done:p0] + fed[:kept]))
            else:
                fill.append((s, p0, fed[:kept]))
            self.filled[id(s)] = p0 + kept
            self.prev[id(s)] = True
        if fill:
            mb = eng.build_batch_explicit(fill)
            self.draft.forward(mb, self.kv, self.states, want_logits=False)

    def draft_batch(self, seqs, k):
        eng = self.eng
        live = [s for s in seqs if id(s) in self.prev]
        if self.hybrid:
            for s in live:
                # recurrent draft models: snapshot the state, draft ahead, restore
                for t_src, t_dst in zip(list(self.states.conv.values()) + list(self.states.ssm.values()),
                                        list(self.state_saved.conv.values()) + list(self.state_saved.ssm.values())):
                    t_dst[s.slot].copy_(t_src[s.slot])
        for s in live:
            s.drafts = []
        for j in range(k):
            items = []
            for s in live:
                pos = len(s.tokens) - 1 + j
                if pos + 2 >= eng.cfg.ctx_size or pos >= s.table.capacity(eng.pool):
                    continue
                items.append((s, pos, [s.tokens[-1] if j == 0 else s.drafts[j - 1]]))
            if not items:
                break
            mb = eng.build_batch_explicit(items)
            o = self.draft.forward(mb, self.kv, self.states)
            for (s, _, _), t in zip(items, ops.argmax(o.logits).tolist()):
                s.drafts.append(int(t))
        if self.hybrid:
            for s in live:
                for t_src, t_dst in zip(list(self.state_saved.conv.values()) + list(self.state_saved.ssm.values()),
                                        list(self.states.conv.values()) + list(self.states.ssm.values())):
                    t_dst[s.slot].copy_(t_src[s.slot])

    def release(self, seq):
        super().release(seq)
        self.filled.pop(id(seq), None)


class Eagle3Config:
    """An EAGLE-3 checkpoint's ``config.json`` (``src/spec/eagle3/config.rs:22-62`` in the reference): the draft
    layer's own shape and the flags that move its norms around."""

    def __init__(self, hidden, n_ff, n_head, n_kv_head, head_dim, vocab, draft_vocab=0, target_hidden=0, n_aux=3,
                 eps=1e-6, rope_theta=10000.0, rope_scaling=None, max_pos=8192, layer_ids=None, attention_bias=False,
                 norm_before_residual=False, norm_before_fc=False, fc_norm=False, norm_output=False, logit_scale=1.0):
        self.hidden, self.n_ff, self.n_head, self.n_kv_head, self.head_dim = hidden, n_ff, n_head, n_kv_head, head_dim
        self.vocab, self.draft_vocab = vocab, draft_vocab or vocab
        self.target_hidden, self.n_aux, self.eps = target_hidden or hidden, n_aux, eps
        self.rope_theta, self.rope_scaling, self.max_pos, self.layer_ids = rope_theta, rope_scaling, max_pos, layer_ids
        self.attention_bias, self.norm_before_residual = attention_bias, norm_before_residual
        self.norm_before_fc, self.fc_norm, self.norm_output, self.logit_scale = norm_before_fc, fc_norm, norm_output, logit_scale
        self.rope_dim = head_dim          # a checkpoint's head rotates its heads whole

    @classmethod
    def for_target(cls, cfg: ModelConfig, draft_vocab: int = 0) -> "Eagle3Config":
        hc = cls(cfg.hidden, cfg.dense_ff or 4 * cfg.hidden, cfg.n_head, cfg.n_kv_head, cfg.head_dim, cfg.vocab,
                 draft_vocab, eps=cfg.rms_eps, rope_theta=cfg.rope_theta, rope_scaling=cfg.rope_scaling,
                 max_pos=cfg.max_position)
        hc.rope_dim = cfg.rope_dim        # a head shaped after the target shares its rotary table
        return hc

    @classmethod
    def parse(cls, c: dict) -> "Eagle3Config":
        if c.get("num_hidden_layers") not in (None, 1):
            raise ValueError(f"config.json: an EAGLE-3 head has one decoder layer, not {c['num_hidden_layers']}")
        if c.get("hidden_act", "silu") != "silu":
            raise ValueError(f"config.json: hidden_act `{c['hidden_act']}` is not supported")
        eagle = c.get("eagle_config") or {}
        if eagle.get("use_aux_hidden_state") is False:
            raise ValueError("config.json: eagle_config.use_aux_hidden_state = false is not supported")
        flag = lambda k: bool(c.get(k, eagle.get(k, False)))          # noqa: E731
        layer_ids = eagle.get("eagle_aux_hidden_state_layer_ids", c.get("eagle_aux_hidden_state_layer_ids"))
        n_aux = c.get("num_aux_hidden_states") or (len(layer_ids) if layer_ids else 3)
        hidden, n_head = int(c["hidden_size"]), int(c["num_attention_heads"])
        rp = c.get("rope_scaling") or c.get("rope_parameters")
        theta = float((rp or {}).get("rope_theta", c.get("rope_theta", 10000.0)))
        if rp and rp.get("rope_type", rp.get("type")) in (None, "default"):
            rp = None
        return cls(hidden, int(c["intermediate_size"]), n_head, int(c.get("num_key_value_heads") or n_head),
                   int(c.get("head_dim") or hidden // n_head), int(c["vocab_size"]), int(c.get("draft_vocab_size") or 0),
                   int(c.get("target_hidden_size") or 0), int(n_aux), float(c.get("rms_norm_eps", 1e-6)), theta, rp,
                   int(c.get("max_position_embeddings", 8192)), [int(v) for v in layer_ids] if layer_ids else None,
                   flag("attention_bias"), flag("norm_before_residual"), flag("norm_before_fc"), flag("fc_norm"),
                   flag("norm_output"), float(c.get("logit_scale", 1.0)))


class Eagle3Head:
    """EAGLE-3 draft head (``src/spec/eagle3/graph.rs:6-16`` in the reference): the target's hidden states of
    ``n_aux`` layers are fused by ``fc`` into one feature g (under ``norm_before_fc`` / ``fc_norm`` behind one norm
    over the concatenation / one per state); the single decoder layer attends over ``[input_layernorm(embed(token)) ;
    hidden_norm(g)]`` rows (input width 2H) with its own KV; h1 = g + o_proj(attention) (the residual is the normed g
    under ``norm_before_residual``), h2 = h1 + mlp(post_attention_layernorm(h1)); logits = lm_head(norm(h2)) over the
    draft vocabulary (mapped back through ``d2t``), times ``logit_scale``; h2 (its normed form under ``norm_output``)
    is g of the next chained step."""

    def __init__(self, cfg: ModelConfig, device, dtype, seed: int = 1, draft_vocab: int = 0, weights=None,
                 hcfg: Optional[Eagle3Config] = None, d2t=None):
        self.cfg = cfg
        self.hc = hc = hcfg or Eagle3Config.for_target(cfg, draft_vocab)
        if hc.hidden != cfg.hidden or hc.vocab != cfg.vocab:
            raise ValueError(f"EAGLE-3 head of width {hc.hidden} / vocabulary {hc.vocab} does not fit a target of width "
                             f"{cfg.hidden} / vocabulary {cfg.vocab} (it reads the target's token embeddings)")
        H, D, nq, nkv, F = hc.hidden, hc.head_dim, hc.n_head, hc.n_kv_head, hc.n_ff
        g = torch.Generator().manual_seed(seed)
        r = lambda *shape: (torch.randn(*shape, generator=g) * 0.02).to(device=device, dtype=dtype)    # noqa: E731
        one = lambda n: torch.ones(n, device=device, dtype=torch.float32)                             # noqa: E731
        self.draft_vocab = hc.draft_vocab
        self.w = weights or {
            "fc": r(H, hc.n_aux * hc.target_hidden), "enorm": one(H), "hnorm": one(H),
            "qkv": r((nq + 2 * nkv) * D, 2 * H), "o": r(H, nq * D), "ffn_norm": one(H), "gate_up": r(2 * F, H),
            "down": r(H, F), "out_norm": one(H), "lm_head": r(self.draft_vocab, H)}
        if d2t is not None:
            self.d2t = d2t.to(device)
        else:
            self.d2t = None if self.draft_vocab == cfg.vocab else torch.arange(self.draft_vocab, device=device)
        self.n_ff = F
        same_rope = (hc.rope_theta == cfg.rope_theta and hc.rope_scaling == cfg.rope_scaling
                     and hc.rope_dim == cfg.rope_dim)
        self.cos_sin = None if same_rope else ops.reference.rope_cos_sin(max(hc.max_pos, cfg.max_position) + 8,
                                                                         hc.rope_dim, hc.rope_theta, hc.rope_scaling,
                                                                         device=device)

    @classmethod
    def from_checkpoint(cls, path: str, cfg: ModelConfig, device, dtype) -> "Eagle3Head":
        """An EAGLE-3 checkpoint directory (``config.json`` + safetensors; decoder layer under ``midlayer.*`` or
        ``layers.0.*``; ``d2t`` offsets when the draft vocabulary is reduced): ``src/spec/eagle3/weights.rs:100-200``."""
        import json
        import os
        from ..loaders.safetensors_io import Checkpoint
        with open(os.path.join(path, "config.json")) as f:
            hc = Eagle3Config.parse(json.load(f))
        ck = Checkpoint(path)
        layer = next((p for p in ("midlayer", "layers.0") if ck.has(f"{p}.input_layernorm.weight")), None)
        if layer is None:
            raise ValueError("the checkpoint has no decoder layer (`midlayer.*` or `layers.0.*`)")

        def get(name, shape=None, f32=False):
            if not ck.has(name):
                raise ValueError(f"the checkpoint has no tensor `{name}`")
            t = ck.get(name)
            if shape is not None and tuple(t.shape) != tuple(shape):
                raise ValueError(f"`{name}` has shape {tuple(t.shape)}, the config needs {tuple(shape)}")
            return t.to(device=device, dtype=torch.float32 if f32 else dtype)

        H, D, nq, nkv, F = hc.hidden, hc.head_dim, hc.n_head, hc.n_kv_head, hc.n_ff
        L = lambda n: f"{layer}.{n}.weight"                                                          # noqa: E731
        w = {"fc": get("fc.weight", (H, hc.n_aux * hc.target_hidden)),
             "qkv": torch.cat([get(L("self_attn.q_proj"), (nq * D, 2 * H)), get(L("self_attn.k_proj"), (nkv * D, 2 * H)),
                               get(L("self_attn.v_proj"), (nkv * D, 2 * H))], 0),
             "o": get(L("self_attn.o_proj"), (H, nq * D)),
             "gate_up": torch.cat([get(L("mlp.gate_proj"), (F, H)), get(L("mlp.up_proj"), (F, H))], 0),
             "down": get(L("mlp.down_proj"), (H, F)), "lm_head": get("lm_head.weight", (hc.draft_vocab, H)),
             "enorm": get(L("input_layernorm"), (H,), True), "hnorm": get(L("hidden_norm"), (H,), True),
             "ffn_norm": get(L("post_attention_layernorm"), (H,), True), "out_norm": get("norm.weight", (H,), True)}
        if hc.norm_before_fc:
            w["input_norm"] = get("input_norm.weight", (hc.n_aux * hc.target_hidden,), True)
        if hc.fc_norm:
            for i in range(hc.n_aux):
                w[f"fc_norm.{i}"] = get(f"fc_norm.{i}.weight", (hc.target_hidden,), True)
        for ours, theirs in (("bq", "self_attn.q_proj.bias"), ("bk", "self_attn.k_proj.bias"),
                             ("bv", "self_attn.v_proj.bias"), ("bo", "self_attn.o_proj.bias"),
                             ("q_norm", "self_attn.q_norm.weight"), ("k_norm", "self_attn.k_norm.weight")):
            if ck.has(f"{layer}.{theirs}"):
                w[ours] = get(f"{layer}.{theirs}", None, True)
        if "bq" in w:
            w["b_qkv"] = torch.cat([w.pop("bq"), w.pop("bk"), w.pop("bv")], 0)
        d2t = None
        if hc.draft_vocab != hc.vocab:
            if not ck.has("d2t"):
                raise ValueError("a reduced draft vocabulary needs the `d2t` map")
            off = ck.get("d2t").long()
            d2t = torch.arange(hc.draft_vocab) + off          # draft id -> target id (the file stores offsets)
            if int(d2t.max()) >= hc.vocab or int(d2t.min()) < 0:
                raise ValueError("`d2t` points outside the target vocabulary")
        return cls(cfg, device, dtype, weights=w, hcfg=hc, d2t=d2t)

    def fuse(self, feats: List[torch.Tensor]) -> torch.Tensor:
        hc, w = self.hc, self.w
        x = torch.cat(feats, dim=-1)
        if hc.norm_before_fc:
            x, _ = ops.rmsnorm(x.contiguous(), w["input_norm"], hc.eps)
        if hc.fc_norm:
            ht = hc.target_hidden
            x = torch.cat([ops.rmsnorm(x[:, i * ht:(i + 1) * ht].contiguous(), w[f"fc_norm.{i}"], hc.eps)[0]
                           for i in range(hc.n_aux)], dim=-1)
        return ops.linear(x.contiguous(), w["fc"])

    def forward(self, tokens_embed, g, b, kv_k, kv_v, cos_sin):
        hc, w = self.hc, self.w
        cos_sin = self.cos_sin if self.cos_sin is not None else cos_sin
        e, _ = ops.rmsnorm(tokens_embed, w["enorm"], hc.eps)
        gn, _ = ops.rmsnorm(g, w["hnorm"], hc.eps)
        x = torch.cat([e, gn], dim=-1).contiguous()
        qkv = ops.linear(x, w["qkv"])
        if "b_qkv" in w:
            qkv = (qkv.float() + w["b_qkv"]).to(qkv.dtype)
        q, _ = ops.qk_norm_rope_append(qkv, hc.n_head, hc.n_kv_head, hc.head_dim, w.get("q_norm"), w.get("k_norm"), hc.eps,
                                       0.0, cos_sin, hc.rope_dim, b.positions, b.slots, kv_k, kv_v, False)
        o = ops.paged_attention(q, kv_k, kv_v, b.block_table, b.ctx_lens, b.cu_q, b.max_q_len, hc.head_dim ** -0.5,
                                max_ctx=b.max_ctx or None)
        h = ops.linear(o.reshape(o.shape[0], -1), w["o"], residual=gn if hc.norm_before_residual else g)
        if "bo" in w:
            h = (h.float() + w["bo"]).to(h.dtype)
        hn, _ = ops.rmsnorm(h, w["ffn_norm"], hc.eps)
        f = ops.linear(ops.gate_up_act(hn, w["gate_up"], self.n_ff), w["down"], residual=h)
        out, _ = ops.rmsnorm(f, w["out_norm"], hc.eps)
        return (out if hc.norm_output else f), out

    def logits(self, normed):
        lg = ops.linear(normed, self.w["lm_head"], out_dtype=torch.float32)
        return lg * self.hc.logit_scale if self.hc.logit_scale != 1.0 else lg


class Eagle3Drafter(_ModelDrafter):
    def __init__(self, engine, head: Optional[Eagle3Head] = None, layer_ids: Optional[List[int]] = None):
        super().__init__(engine)
        cfg = engine.mcfg
        n = cfg.n_layer
        self.head = head or Eagle3Head(cfg, engine.device, engine.model.dtype)
        hc = self.head.hc
        self.capture_layers = layer_ids or hc.layer_ids or sorted({min(2, n - 1), n // 2, max(0, n - 3)})
        while len(self.capture_layers) < hc.n_aux:
            self.capture_layers = sorted(set(self.capture_layers) | {len(self.capture_layers)})[:hc.n_aux] \
                if n >= hc.n_aux else (self.capture_layers + [self.capture_layers[-1]])
        if max(self.capture_layers) >= n:
            raise ValueError(f"the EAGLE-3 head reads target layers {self.capture_layers}, the target has {n}")
        nb = engine.pool.total
        shape = (nb, engine.cfg.block_size, hc.n_kv_head, hc.head_dim)
        self.k = torch.zeros(shape, device=engine.device, dtype=engine.model.dtype)
        self.v = torch.zeros(shape, device=engine.device, dtype=engine.model.dtype)

    def _features(self, out, lo, hi):
        return self.head.fuse([out.captures[l][lo:hi] for l in self.capture_layers[:self.head.hc.n_aux]])

    def on_step(self, items, b, out):
        eng = self.eng
        cu = b.cu_q_host
        fill, gs = [], []
        for s, p0, fed, kept, bi in items:
            if kept <= 0:
                continue
            g_rows = self._features(out, cu[bi], cu[bi] + kept)      # g_p for positions p0 .. p0+kept-1
            first = self.prev.get(id(s))
            if first is None:
                first = self._zeros(eng.mcfg.hidden)
            # the row for position p pairs token p with the feature of position p - 1
            gs.append(torch.cat([first[None], g_rows[:kept - 1]], dim=0))
            fill.append((s, p0, fed[:kept]))
            self.prev[id(s)] = g_rows[kept - 1].clone()
        if fill:
            mb = eng.build_batch_explicit(fill)
            self.head.forward(eng.model.embed(mb.token_ids), torch.cat(gs, dim=0), mb, self.k, self.v, eng.model.cos_sin)

    def draft_batch(self, seqs, k):
        eng = self.eng
        live = [s for s in seqs if id(s) in self.prev]
        for s in live:
            s.drafts = []
        feat = {id(s): self.prev[id(s)] for s in live}
        for j in range(k):
            items, gs = [], []
            for s in live:
                pos = len(s.tokens) - 1 + j
                if pos + 2 >= eng.cfg.ctx_size or pos >= s.table.capacity(eng.pool):
                    continue
                items.append((s, pos, [s.tokens[-1] if j == 0 else s.drafts[j - 1]]))
                gs.append(feat[id(s)][None])
            if not items:
                break
            mb = eng.build_batch_explicit(items)
            raw, normed = self.head.forward(eng.model.embed(mb.token_ids), torch.cat(gs, dim=0), mb, self.k, self.v,
                                            eng.model.cos_sin)
            picks = ops.argmax(self.head.logits(normed))
            if self.head.d2t is not None:
                picks = self.head.d2t[picks.long()]
            for (s, _, _), t, row in zip(items, picks.tolist(), raw):
                s.drafts.append(int(t))
                feat[id(s)] = row


class DflashDrafter(_ModelDrafter):
    """Block drafter: ONE pass proposes a whole block of k tokens from the target's last hidden row. Each
    block position j gets ``proj(h) + pos_emb[j]``; one bidirectional self-attention layer over the block and
    an FFN mix the positions; the target's LM head scores them (``src/spec/dflash.rs:1-75``: one pass per
    block, no chaining)."""

    def __init__(self, engine, block: int = 8, seed: int = 2):
        super().__init__(engine)
        cfg = engine.mcfg
        H = cfg.hidden
        g = torch.Generator().manual_seed(seed)
        r = lambda *shape: (torch.randn(*shape, generator=g) * 0.02).to(device=engine.device, dtype=engine.model.dtype)
        self.block = block
        self.w = {"proj": r(H, H), "pos": r(block, H), "qkv": r(3 * H, H), "o": r(H, H), "gate_up": r(4 * H, H),
                  "down": r(H, 2 * H), "norm": torch.ones(H, device=engine.device)}

    def on_step(self, items, b, out):
        cu = b.cu_q_host
        for s, p0, fed, kept, bi in items:
            if kept > 0:
                self.prev[id(s)] = out.last_hidden[cu[bi] + kept - 1].clone()

    def draft_batch(self, seqs, k):
        eng = self.eng
        live = [s for s in seqs if id(s) in self.prev]
        if not live:
            return
        k = min(k, self.block)
        w = self.w
        H = eng.mcfg.hidden
        h = torch.stack([self.prev[id(s)] for s in live])                       # [n, H]
        x = (ops.linear(h, w["proj"]).float()[:, None, :] + w["pos"][:k].float()[None]).to(h.dtype)   # [n, k, H]
        n = x.shape[0]
        qkv = ops.linear(x.reshape(n * k, H), w["qkv"]).float().view(n, k, 3, H)
        att = torch.softmax(qkv[:, :, 0] @ qkv[:, :, 1].transpose(1, 2) * H ** -0.5, dim=-1) @ qkv[:, :, 2]
        y = ops.linear(att.reshape(n * k, H).to(h.dtype), w["o"], residual=x.reshape(n * k, H))
        f = ops.linear(ops.gate_up_act(y, w["gate_up"], 2 * H), w["down"], residual=y)
        normed, _ = ops.rmsnorm(f, w["norm"], eng.mcfg.rms_eps)
        picks = ops.argmax(eng.model.logits(normed)).view(n, k).tolist()
        for s, p in zip(live, picks):
            room = eng.cfg.ctx_size - len(s.tokens) - 2
            s.drafts = [int(t) for t in p[:max(0, room)]]
