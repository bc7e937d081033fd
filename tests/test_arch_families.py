"""Architecture families built from optional blocks: hyper-connections (both forms), Kimi delta attention, latent
MoE with un-gated experts. The vectorised forms against token-serial restatements of the reference's definitions, and
the engine invariants on tiny models of each family (CPU, fp32)."""
import math

import pytest
import torch

from legion_b200.config import PRESETS
from legion_b200.engine.lm import EngineConfig, build_engine
from legion_b200.models.decoder import Decoder, KvCache, StatePool, StepBatch
from legion_b200.models.weights import random_weights


def _model(seed=1):
    cfg = PRESETS["tiny-glm-next"]()
    w = random_weights(cfg, "cpu", torch.float32, seed=seed, std=0.08)
    return cfg, w, Decoder(cfg, w, None, max_position=300)


def test_hyper_connection_mixer_matches_the_serial_definition():
    cfg, w, m = _model()
    T, hc, H = 5, cfg.hyper_streams, cfg.hidden
    X = torch.randn(T, hc, H)
    y, post, comb = m._hc_pre("l0.hca", X)
    f, scale, base = w["l0.hca.hc_f"], w["l0.hca.hc_scale"], w["l0.hca.hc_base"]
    eps = cfg.hc_eps
    sig = lambda v: 1 / (1 + math.exp(-v))      # noqa: E731
    for t in range(T):
        flat = X[t].reshape(-1)
        normed = flat / math.sqrt(float(flat.pow(2).mean()) + cfg.rms_eps)
        mix = (f @ normed).tolist()
        pre = [sig(mix[h] * float(scale[0]) + float(base[h])) + eps for h in range(hc)]
        po = [sig(mix[hc + h] * float(scale[1]) + float(base[hc + h])) * 2 for h in range(hc)]
        c = [mix[2 * hc + i] * float(scale[2]) + float(base[2 * hc + i]) for i in range(hc * hc)]    # c[d + hc * s]
        for s in range(hc):
            col = c[s * hc:(s + 1) * hc]
            mx = max(col)
            ex = [math.exp(v - mx) for v in col]
            tot = sum(ex)
            c[s * hc:(s + 1) * hc] = [v / tot + eps for v in ex]

        def cols():
            for d in range(hc):
                sm = sum(c[d + hc * s] for s in range(hc)) + eps
                for s in range(hc):
                    c[d + hc * s] /= sm

        def rows():
            for s in range(hc):
                sm = sum(c[s * hc:(s + 1) * hc]) + eps
                for d in range(hc):
                    c[s * hc + d] /= sm
        cols()
        for _ in range(1, cfg.hc_iters):
            rows()
            cols()
        assert torch.allclose(post[t], torch.tensor(po), atol=1e-5)
        want_y = sum(X[t, h] * pre[h] for h in range(hc))
        assert torch.allclose(y[t], want_y, atol=1e-5)
        for d in range(hc):
            for s in range(hc):
                assert abs(float(comb[t, d, s]) - c[d + hc * s]) < 1e-5
        # the mix is (close to) doubly stochastic after the Sinkhorn rounds
        assert torch.allclose(comb[t].sum(1), torch.ones(hc), atol=1e-2)
    out = torch.randn(T, H)
    new = Decoder._hc_post(out, X, post, comb)
    d, t = 2, 3
    want = out[t] * post[t, d] + sum(X[t, s] * comb[t, d, s] for s in range(hc))
    assert torch.allclose(new[t, d], want, atol=1e-5)


def test_kimi_delta_attention_matches_the_token_serial_recurrence():
    cfg, w, m = _model(seed=2)
    nh, d, KC = cfg.kda_heads, cfg.kda_head_dim, cfg.kda_conv
    c = nh * d
    lens = [7, 1, 4]
    T = sum(lens)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    x = torch.randn(T, cfg.hidden) * 0.5
    st = StatePool(cfg, 4, "cpu")
    st.conv[0].normal_(0, 0.3)
    st.ssm[0].normal_(0, 0.3)
    conv0, ssm0 = st.conv[0].clone(), st.ssm[0].clone()
    slots = [2, 0, 3]
    i32 = dict(dtype=torch.int32)
    b = StepBatch(token_ids=torch.zeros(T, **i32), positions=torch.zeros(T, **i32), cu_q=torch.tensor(cu, **i32),
                  ctx_lens=torch.tensor(lens, **i32), block_table=torch.zeros(3, 1, **i32),
                  slots=torch.zeros(T, dtype=torch.int64), state_slots=torch.tensor(slots, **i32), max_q_len=max(lens),
                  cu_q_host=cu)
    got = m._kda("l0", 0, x, b, st)
    p = "l0.kda"
    qkv = x @ w[f"{p}.qkv"].t()
    z = (x @ w[f"{p}.f_a"].t()) @ w[f"{p}.f_b"].t()
    gate = (x @ w[f"{p}.g_a"].t()) @ w[f"{p}.g_b"].t()
    beta = torch.sigmoid(x @ w[f"{p}.beta"].t())
    want = torch.zeros(T, c)
    for si, n in enumerate(lens):
        hist = conv0[slots[si]].clone()              # [3c, KC - 1]
        S = ssm0[slots[si]].clone()                  # [heads, j, i]
        for t in range(cu[si], cu[si] + n):
            win = torch.cat([hist, qkv[t].unsqueeze(1)], 1)
            y = (win * w[f"{p}.conv_w"]).sum(1)
            y = y * torch.sigmoid(y)
            hist = win[:, 1:]
            for h in range(nh):
                q, k, v = (y[j * c + h * d:j * c + (h + 1) * d] for j in range(3))
                qn = q * (d ** -0.5) / torch.sqrt(q.pow(2).sum() + 1e-6)
                kn = k / torch.sqrt(k.pow(2).sum() + 1e-6)
                g = cfg.kda_lower * torch.sigmoid(-((z[t, h * d:(h + 1) * d] + w[f"{p}.dt_bias"][h * d:(h + 1) * d])
                                                    * w[f"{p}.A"][h]))
                for j in range(d):
                    row = S[h, j] * g.exp()
                    delta = (v[j] - row @ kn) * beta[t, h]
                    row = row + delta * kn
                    S[h, j] = row
                    want[t, h * d + j] = row @ qn
        assert torch.allclose(st.conv[0][slots[si]], hist, atol=1e-5)
        assert torch.allclose(st.ssm[0][slots[si]], S, atol=1e-4)
    o = want.view(T, nh, d)
    o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * w[f"{p}.norm"]
    o = (o * torch.sigmoid(gate.view(T, nh, d))).reshape(T, c) @ w[f"{p}.out"].t()
    assert torch.allclose(got, o, atol=2e-4, rtol=1e-3)
    assert torch.equal(st.ssm[0][1], ssm0[1])        # an unused slot is untouched


def test_engine_invariants_on_the_tiny_glm_next_model():
    """Batched == single, chunked prefill == one pass (recurrent state carried between chunks), and a repeated
    prompt resumes from the prefix cache with its recurrent snapshot."""
    cfg = PRESETS["tiny-glm-next"]()
    w = random_weights(cfg, "cpu", torch.float32, seed=3, std=0.08)
    ec = dict(ctx_size=256, max_seqs=4, block_size=16, max_batch_tokens=256)
    prompts = [list(range(5, 5 + n)) for n in (41, 23, 60)]
    one = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(prefill_chunk=256, **ec))
    singles = [one.generate_text(tokens=p, max_tokens=6, ignore_eos=True).token_ids for p in prompts]
    again = one.generate_text(tokens=prompts[2], max_tokens=6, ignore_eos=True)
    one.shutdown()
    assert again.token_ids == singles[2] and again.usage.cached_tokens >= 16
    chunked = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(prefill_chunk=16, **ec))
    streams = [chunked.generate(__import__("legion_b200.engine.types", fromlist=["GenerateRequest"]).GenerateRequest(
        prompt_tokens=p, sampling=__import__("legion_b200.engine.types", fromlist=["SamplingParams"]).SamplingParams(
            max_tokens=6, ignore_eos=True))) for p in prompts]
    outs = [s.collect().token_ids for s in streams]
    chunked.shutdown()
    assert outs == singles


def test_gated_hyper_connections_match_the_serial_definition_and_the_engine_invariants_hold():
    """qwen4exp's mixer: per-stream RMS norm, low-rank sigmoid gate, mean of the gated streams; the block output
    re-enters stream h with 2 sigmoid(inject[h] / hc). Then the engine on the tiny model of that family: batched ==
    single, chunked prefill == one pass, n-gram speculation == plain decoding (recurrent state replayed)."""
    cfg = PRESETS["tiny-qwen4exp"]()
    w = random_weights(cfg, "cpu", torch.float32, seed=5, std=0.08)
    assert "l0.attn_norm" not in w and "output_norm" not in w and "out_hc.hcg_up" in w
    m = Decoder(cfg, w, None, max_position=300)
    T, hc, H = 4, cfg.hyper_streams, cfg.hidden
    X = torch.randn(T, hc, H)
    y, inj = m._hcg_mix("l1.hcf", X, True)
    nw, dn, up, ij = (w[f"l1.hcf.hcg_{k}"] for k in ("norm", "down", "up", "inject"))
    for t in range(T):
        xn = torch.stack([X[t, s] / torch.sqrt(X[t, s].pow(2).mean() + cfg.rms_eps) * nw[s] for s in range(hc)])
        flat = xn.reshape(-1)
        lo = torch.nn.functional.silu((dn @ flat) / hc)
        gate = (up @ lo).view(hc, H)
        want = sum(xn[s] * torch.sigmoid(gate[s]) for s in range(hc)) / hc
        assert torch.allclose(y[t], want, atol=1e-5)
        assert torch.allclose(inj[t], ij @ flat, atol=1e-5)
    out = torch.randn(T, H)
    new = Decoder._hcg_combine(out, X, inj)
    assert torch.allclose(new[2, 1], X[2, 1] + out[2] * 2 * torch.sigmoid(inj[2, 1] / hc), atol=1e-6)
    ec = dict(ctx_size=256, max_seqs=4, block_size=16, max_batch_tokens=256)
    prompts = [list(range(5, 5 + n)) + [7, 8, 9, 7, 8, 9, 7, 8] for n in (33, 18)]
    one = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(prefill_chunk=256, **ec))
    singles = [one.generate_text(tokens=p, max_tokens=8, ignore_eos=True).token_ids for p in prompts]
    one.shutdown()
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    for kw in (dict(prefill_chunk=16), dict(prefill_chunk=256, spec="ngram", spec_k=3)):
        eng = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(**kw, **ec))
        streams = [eng.generate(GenerateRequest(prompt_tokens=p, sampling=SamplingParams(max_tokens=8, ignore_eos=True)))
                   for p in prompts]
        outs = [s.collect().token_ids for s in streams]
        eng.shutdown()
        assert outs == singles, kw


def test_latent_moe_with_ungated_experts():
    """Nemotron-H's MoE: router on the full-width input, squared-ReLU experts between a down and an up projection,
    shared expert at full width. The layer against a direct restatement; batched == single, chunked == one pass."""
    cfg = PRESETS["tiny-nemotron-h-moe"]()
    w = random_weights(cfg, "cpu", torch.float32, seed=6, std=0.08)
    assert w["l1.moe.gate_up"].shape == (8, 128, 128) and w["l1.moe.lat_down"].shape == (128, 256)
    m = Decoder(cfg, w, None, max_position=300)
    x = torch.randn(5, cfg.hidden) * 0.5
    out, fused, _ = m._ffn("l1", True, x, None)
    logits = x @ w["l1.moe.router"].t()
    sc = torch.sigmoid(logits)
    top = torch.topk(sc + w["l1.moe.router_bias"], cfg.top_k, dim=-1).indices
    want = torch.zeros_like(x)
    xl = x @ w["l1.moe.lat_down"].t()
    for t in range(5):
        ws = sc[t, top[t]]
        ws = ws / ws.sum() * cfg.route_scale
        acc = torch.zeros(cfg.moe_latent)
        for e, wt in zip(top[t].tolist(), ws.tolist()):
            h = torch.relu(w["l1.moe.gate_up"][e] @ xl[t]) ** 2
            acc += wt * (w["l1.moe.down"][e] @ h)
        sh = w["l1.moe.sh_down"] @ (torch.relu(w["l1.moe.sh_gate_up"] @ x[t]) ** 2)
        want[t] = w["l1.moe.lat_up"] @ acc + sh
    assert not fused and torch.allclose(out, want, atol=2e-4, rtol=1e-3)
    ec = dict(ctx_size=256, max_seqs=4, block_size=16, max_batch_tokens=256)
    prompts = [list(range(5, 5 + n)) for n in (37, 20)]
    one = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(prefill_chunk=256, **ec))
    singles = [one.generate_text(tokens=p, max_tokens=6, ignore_eos=True).token_ids for p in prompts]
    one.shutdown()
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    eng = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(prefill_chunk=16, **ec))
    streams = [eng.generate(GenerateRequest(prompt_tokens=p, sampling=SamplingParams(max_tokens=6, ignore_eos=True)))
               for p in prompts]
    outs = [s.collect().token_ids for s in streams]
    eng.shutdown()
    assert outs == singles


def test_gemma4_layer_form_against_a_plain_restatement():
    """The Gemma-4 forward (sandwich norms, scaled embedding, per-kind head sizes / kv heads / rotary tables, value
    norm, keys as values on global layers, shared KV layers, dense FFN beside routed GELU experts, per-layer
    embeddings, output scale, soft cap) against a cache-free restatement in plain tensor operations; then the engine
    invariants (batched == single, chunked prefill == one pass, prefix-cache resume) on the same model."""
    import torch.nn.functional as F
    cfg = PRESETS["tiny-gemma4"]()
    w = random_weights(cfg, "cpu", torch.float32, seed=8, std=0.06)
    w = {k: (v + 0.1 * torch.randn_like(v) if k.endswith("norm") else v) for k, v in w.items()}
    toks = list(range(11, 11 + 70))              # longer than the 48-token window
    T, H, L, npl = len(toks), cfg.hidden, cfg.n_layer, cfg.ple_dim
    eps = cfg.rms_eps

    def rms(t, wt=None):
        y = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps)
        return y if wt is None else y * wt

    def rope(t, theta, rot, factors=None):
        half = rot // 2
        inv = 1.0 / (theta ** (torch.arange(half, dtype=torch.float64) / half))
        if factors is not None:
            inv = inv / torch.tensor(factors, dtype=torch.float64)
        ang = torch.arange(T, dtype=torch.float64)[:, None] * inv[None]
        c, s_ = ang.cos().float()[:, None, :], ang.sin().float()[:, None, :]
        a, b = t[..., :half], t[..., half:rot]
        return torch.cat([a * c - b * s_, b * c + a * s_, t[..., rot:]], -1)

    ids = torch.tensor(toks)
    x = w["tok_embd"][ids] * cfg.embed_scale
    rows = w["ple_embd"][ids] * npl ** 0.5
    pr = ((x @ w["ple_model_proj"].t()) * H ** -0.5).view(T, L, npl)
    ple = (rms(pr, w["ple_proj_norm"]) + rows.view(T, L, npl)) * 2 ** -0.5
    kv_of = {}
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for il in range(L):
        p = f"l{il}"
        swa = cfg.layer_kinds[il] == "swa"
        D, n_kv = cfg.attn_dims(il)
        nh = cfg.n_head
        h = rms(x, w[f"{p}.attn_norm"])
        proj = h @ w[f"{p}.attn.qkv"].t()
        q = rms(proj[:, :nh * D].view(T, nh, D), w[f"{p}.attn.q_norm"])
        theta, rot, fac = (cfg.rope_theta_swa, D, None) if swa else (cfg.rope_theta, cfg.rope_dim, cfg.rope_freq_factors)
        q = rope(q, theta, rot, fac)
        if cfg.owns_kv(il):
            kraw = proj[:, nh * D:(nh + n_kv) * D].view(T, n_kv, D)
            vraw = proj[:, (nh + n_kv) * D:].view(T, n_kv, D) if cfg.has_v_proj(il) else kraw
            kv_of[il] = (rope(rms(kraw, w[f"{p}.attn.k_norm"]), theta, rot, fac), rms(vraw))
        k, v = kv_of[cfg.kv_source(il)]
        rep = nh // n_kv
        sc = torch.einsum("qhd,khd->hqk", q, k.repeat_interleave(rep, 1))          # unscaled
        mask = causal.clone()
        if swa:
            mask &= ~torch.tril(torch.ones(T, T, dtype=torch.bool), -cfg.sliding_window)
        o = torch.einsum("hqk,khd->qhd", torch.softmax(sc.masked_fill(~mask[None], float("-inf")), -1),
                         v.repeat_interleave(rep, 1)).reshape(T, nh * D)
        attn_out = rms(o @ w[f"{p}.attn.o"].t(), w[f"{p}.attn_post_norm"]) + x
        hh = rms(attn_out, w[f"{p}.ffn_norm"]) @ w[f"{p}.mlp.gate_up"].t()
        Fd = cfg.dense_ff
        mlp = (F.gelu(hh[:, :Fd], approximate="tanh") * hh[:, Fd:]) @ w[f"{p}.mlp.down"].t()
        if cfg.is_moe_layer(il):
            mlp = rms(mlp, w[f"{p}.ffn_post1_norm"])
            r = rms(attn_out) * H ** -0.5 * w[f"{p}.moe.router_scale"]
            probs = torch.softmax(r @ w[f"{p}.moe.router"].t(), -1)
            tw, ti = torch.topk(probs, cfg.top_k, -1)
            tw = tw / tw.sum(-1, keepdim=True)
            moe_in = rms(attn_out, w[f"{p}.ffn_pre2_norm"])
            y = torch.zeros(T, H)
            Fe = cfg.expert_ff
            for t in range(T):
                for e, wt in zip(ti[t].tolist(), tw[t].tolist()):
                    g = w[f"{p}.moe.gate_up"][e] @ moe_in[t]
                    y[t] += wt * (w[f"{p}.moe.down"][e] @ (F.gelu(g[:Fe], approximate="tanh") * g[Fe:]))
            mlp = mlp + rms(y, w[f"{p}.ffn_post2_norm"])
        cur = rms(mlp, w[f"{p}.ffn_post_norm"]) + attn_out
        t_ = F.gelu(cur @ w[f"{p}.ple.inp_gate"].t(), approximate="tanh") * ple[:, il]
        cur = cur + rms(t_ @ w[f"{p}.ple.proj"].t(), w[f"{p}.ple.post_norm"])
        x = cur * w[f"{p}.out_scale"]
    lg = rms(x, w["output_norm"]) @ w["tok_embd"].t()
    want = torch.tanh(lg / cfg.logit_softcap) * cfg.logit_softcap

    ec = dict(ctx_size=256, max_seqs=4, block_size=16, max_batch_tokens=256)
    eng = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(prefill_chunk=256, **ec), start=False)
    assert eng.kv.k[5] is eng.kv.k[2] and eng.kv.k[4] is eng.kv.k[3] and eng.kv.k[0].shape[2:] == (2, 64)
    assert eng.kv.k[2].shape[2:] == (1, 128)
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    seq = eng.prepare(GenerateRequest(prompt_tokens=toks, sampling=SamplingParams(max_tokens=1)))
    eng.waiting.push(seq)
    eng._admit()
    b = eng.build_batch([(seq, 0, T)])
    b.logit_rows = None
    got = eng.model.forward(b, eng.kv, eng.states).logits
    assert torch.allclose(got, want, atol=3e-3, rtol=1e-3), float((got - want).abs().max())

    prompts = [list(range(5, 5 + n)) for n in (75, 23, 60)]
    one = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(prefill_chunk=256, **ec))
    singles = [one.generate_text(tokens=p_, max_tokens=6, ignore_eos=True).token_ids for p_ in prompts]
    again = one.generate_text(tokens=prompts[0], max_tokens=6, ignore_eos=True)
    one.shutdown()
    assert again.token_ids == singles[0] and again.usage.cached_tokens >= 16
    for kw in (dict(prefill_chunk=16), dict(prefill_chunk=32, kv_rings=True, prefix_cache=False)):
        eng2 = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(**kw, **ec))
        streams = [eng2.generate(GenerateRequest(prompt_tokens=p_, sampling=SamplingParams(max_tokens=6, ignore_eos=True)))
                   for p_ in prompts]
        outs = [s_.collect().token_ids for s_ in streams]
        ring = eng2.ring_len
        eng2.shutdown()
        assert outs == singles, kw
        assert (ring > 0) == bool(kw.get("kv_rings"))


def test_gemma4_gguf_round_trip(tmp_path):
    """The Gemma-4 layer form written as a ``gemma4`` GGUF (keys and tensor names as the reference reads them) and
    read back: same configuration, same tensors, same tokens."""
    from legion_b200.loaders.gguf_map import load_gguf, write_gguf
    cfg = PRESETS["tiny-gemma4"]()
    w = random_weights(cfg, "cpu", torch.float32, seed=8, std=0.06)
    path = str(tmp_path / "gemma4.gguf")
    write_gguf(path, cfg, w)
    cfg2, w2, md = load_gguf(path)
    assert md["general.architecture"] == "gemma4" and md["gemma4.attention.shared_kv_layers"] == 2
    for f in ("layer_kinds", "kv_shared_layers", "global_k_as_v", "layer_out_scale", "first_dense_layers", "n_expert",
              "ple_dim", "swa_head_dim", "swa_kv_heads", "n_kv_head", "head_dim", "sliding_window", "logit_softcap",
              "rope_theta_swa", "sandwich_norm", "v_norm", "embed_scale", "attn_scale"):
        assert getattr(cfg2, f) == getattr(cfg, f), f
    assert cfg2.rope_freq_factors == cfg.rope_freq_factors
    assert set(w2) == set(w) and all(torch.allclose(w[k].float(), w2[k].float()) for k in w)
    ec = dict(ctx_size=256, max_seqs=2, block_size=16, max_batch_tokens=128)
    toks = list(range(9, 80))
    outs = []
    for c, ww in ((cfg, w), (cfg2, w2)):
        eng = build_engine(c, weights=dict(ww), engine_cfg=EngineConfig(**ec))
        outs.append(eng.generate_text(tokens=toks, max_tokens=8, ignore_eos=True).token_ids)
        eng.shutdown()
    assert outs[0] == outs[1]


@pytest.mark.parametrize("variant", ["dense", "moe"])
def test_gemma4_hf_checkpoint_against_transformers(tmp_path, variant):
    """A tiny Gemma-4 text model built and saved by the ``transformers`` implementation, read through the HF mapper
    (``loaders/hf_gemma4.py``): the prompt's logits at every position and a greedy continuation match that
    implementation. dense: per-layer embeddings, layers that share KV and are twice as wide, proportional rotary
    embedding on the global layers, a window shorter than the prompt, soft cap. moe: routed experts beside the dense
    FFN with a per-expert output scale, keys as values and a kv-head count of their own on the global layers."""
    g4 = pytest.importorskip("transformers.models.gemma4.modeling_gemma4")
    from transformers.models.gemma4 import Gemma4TextConfig
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    from legion_b200.loaders.hf_map import load_hf
    torch.manual_seed(0)
    kw = dict(vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=6, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, global_head_dim=32, sliding_window=8,
              layer_types=["sliding_attention", "sliding_attention", "full_attention"] * 2,
              vocab_size_per_layer_input=320, hidden_size_per_layer_input=8, num_kv_shared_layers=2,
              final_logit_softcapping=30.0, max_position_embeddings=256, use_double_wide_mlp=True,
              attention_k_eq_v=False, pad_token_id=0, eos_token_id=1, bos_token_id=2)
    if variant == "moe":
        kw.update(enable_moe_block=True, num_experts=8, top_k_experts=2, moe_intermediate_size=32,
                  num_kv_shared_layers=0, hidden_size_per_layer_input=0, attention_k_eq_v=True,
                  num_global_key_value_heads=1, use_double_wide_mlp=False)
    hc = Gemma4TextConfig(**kw)
    hc._attn_implementation = "eager"
    m = g4.Gemma4ForCausalLM(hc).eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" in n or n.endswith("router.scale") or n.endswith("per_expert_scale"):
                p.copy_(1.0 + 0.2 * torch.randn_like(p))
            elif p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.08)
        for n, b in m.named_buffers():
            if n.endswith("layer_scalar"):
                b.copy_(torch.tensor([0.9]))
    m.save_pretrained(str(tmp_path), safe_serialization=True)
    ids = torch.randint(3, 320, (1, 24))
    with torch.no_grad():
        ref = m(input_ids=ids).logits[0].float()
        cont = m.generate(ids, max_new_tokens=6, do_sample=False)[0, 24:].tolist()
    cfg, w, _ = load_hf(str(tmp_path), "cpu", torch.float32)
    assert cfg.sandwich_norm and cfg.layer_kinds == ["swa", "swa", "attn"] * 2
    assert cfg.global_k_as_v == (variant == "moe") and cfg.n_expert == (8 if variant == "moe" else 0)
    eng = build_engine(cfg, weights=dict(w), start=False,
                       engine_cfg=EngineConfig(ctx_size=128, max_seqs=2, block_size=16, max_batch_tokens=128))
    seq = eng.prepare(GenerateRequest(prompt_tokens=ids[0].tolist(), sampling=SamplingParams(max_tokens=1)))
    eng.waiting.push(seq)
    eng._admit()
    b = eng.build_batch([(seq, 0, 24)])
    b.logit_rows = None
    with torch.no_grad():
        mine = eng.model.forward(b, eng.kv, eng.states).logits.float()
    assert (mine - ref).abs().max().item() < 2e-4
    eng2 = build_engine(cfg, weights=dict(w),
                        engine_cfg=EngineConfig(ctx_size=128, max_seqs=2, block_size=16, max_batch_tokens=128,
                                                prefill_chunk=16))
    out = eng2.generate_text(tokens=ids[0].tolist(), max_tokens=6, ignore_eos=True).token_ids
    eng2.shutdown()
    assert out == cont


def test_block_form_engine_invariants():
    """One sub-layer per block (Nemotron-H as shipped), including a dense FFN block: batched == single, chunked
    prefill == one pass, and a repeated prompt resumes from the prefix cache's state snapshots."""
    cfg = PRESETS["tiny-nemotron-h-blocks"]()
    w = random_weights(cfg, "cpu", torch.float32, seed=3, std=0.05)
    assert "l1.mlp.down" in w and "l1.attn.qkv" not in w and "l0.mlp.down" not in w and "l3.moe.lat_down" in w
    ec = dict(ctx_size=256, max_seqs=4, block_size=16, max_batch_tokens=128)
    eng = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(**ec))
    prompts = [list(range(5 + i, 75 + 3 * i)) for i in range(3)]
    single = [eng.generate_text(tokens=p, max_tokens=10, ignore_eos=True).token_ids for p in prompts]
    import threading
    got = [None] * 3

    def go(i):
        got[i] = eng.generate_text(tokens=prompts[i], max_tokens=10, ignore_eos=True).token_ids

    ts = [threading.Thread(target=go, args=(i,)) for i in range(3)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    r = eng.generate_text(tokens=prompts[0], max_tokens=10, ignore_eos=True)
    eng.shutdown()
    assert got == single and r.token_ids == single[0] and r.usage.cached_tokens > 0
    eng2 = build_engine(cfg, weights=dict(w), engine_cfg=EngineConfig(prefill_chunk=16, prefix_cache=False, **ec))
    chunked = eng2.generate_text(tokens=prompts[1], max_tokens=10, ignore_eos=True).token_ids
    eng2.shutdown()
    assert chunked == single[1]


def test_nemotron_h_blocks_gguf_round_trip(tmp_path):
    """The block form as a ``nemotron_h_moe`` GGUF (per-layer kv-head and FFN-size arrays tell the block kinds; tensor
    names from llama.cpp's table, checked against the ``gguf`` package when it is there): same configuration, same
    tensors, same tokens."""
    import re
    from legion_b200.loaders.gguf_map import load_gguf, to_gguf_tensors, write_gguf
    cfg = PRESETS["tiny-nemotron-h-blocks"]()
    w = random_weights(cfg, "cpu", torch.float32, seed=3, std=0.05)
    path = str(tmp_path / "nh.gguf")
    write_gguf(path, cfg, w)
    cfg2, w2, md = load_gguf(path)
    assert md["general.architecture"] == "nemotron_h_moe" and cfg2.block_form
    for f in ("layer_kinds", "n_expert", "top_k", "expert_ff", "shared_ff", "moe_latent", "ssm_groups", "ssm_heads",
              "ssm_head_dim", "ssm_state", "n_kv_head", "head_dim", "router_mode", "norm_topk", "route_scale"):
        assert getattr(cfg2, f) == getattr(cfg, f), f
    assert set(w2) == set(w) and all(torch.allclose(w[k].float(), w2[k].float()) for k in w)
    try:
        import gguf
        arch = {v: k for k, v in gguf.MODEL_ARCH_NAMES.items()}["nemotron_h_moe"]
        allowed = {gguf.TENSOR_NAMES[t] for t in gguf.MODEL_TENSORS[arch]}
        for n in to_gguf_tensors(cfg, w):
            assert re.sub(r"\.(weight|bias)$", "", re.sub(r"^blk\.\d+\.", "blk.{bid}.", n)) in allowed, n
    except ImportError:
        pass
    ec = dict(ctx_size=256, max_seqs=2, block_size=16, max_batch_tokens=128)
    outs = []
    for c, ww in ((cfg, w), (cfg2, w2)):
        eng = build_engine(c, weights=dict(ww), engine_cfg=EngineConfig(**ec))
        outs.append(eng.generate_text(tokens=list(range(9, 70)), max_tokens=8, ignore_eos=True).token_ids)
        eng.shutdown()
    assert outs[0] == outs[1]
