"""Plain PyTorch reference of every op (the oracle for the sm_100a kernels and the CPU back-end).

All math is done in float32 whatever the input dtype; outputs are cast back to the input dtype.
Shapes follow the kernel interfaces: activations are token-major ``[T, features]``, the paged KV
cache is ``[blocks, page, kv_heads, head_dim]`` and a block table row lists a sequence's blocks.
Reference counterparts: the CPU implementation of each external op in the reference engine
(``src/model/core/*.rs`` ``cpu`` functions, e.g. ``src/model/core/gdn_scan.rs:195-262``).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def rmsnorm(x, w, eps: float, w_offset: float = 0.0, residual=None):
    """Returns (normed, summed) where summed = x (+ residual)."""
    xf = x.float()
    if residual is not None:
        xf = (xf + residual.float()).to(x.dtype).float()
    summed = xf.to(x.dtype)
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = xf * inv * (w.float() + w_offset)
    return y.to(x.dtype), summed


def linear(x, w, residual=None, out_dtype=None):
    y = x.float() @ w.float().t()
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype or x.dtype)


def gate_up_act(x, w_gate_up, n_ff: int, act: str = "silu"):
    """w_gate_up rows: [gate(n_ff) | up(n_ff)]; returns act(gate) * up."""
    h = x.float() @ w_gate_up.float().t()
    if w_gate_up.shape[0] == n_ff:            # un-gated FFN (squared ReLU): only the up projection exists
        return activation(h, act).to(x.dtype)
    g, u = h[:, :n_ff], h[:, n_ff:2 * n_ff]
    return (activation(g, act) * u).to(x.dtype)


def activation(g, act: str):
    if act == "silu":
        return F.silu(g)
    if act == "gelu_tanh":
        return F.gelu(g, approximate="tanh")
    if act == "relu2":
        return F.relu(g).pow(2)
    raise ValueError(act)


def rope_cos_sin(max_pos: int, rot: int, theta: float, scaling: Optional[dict] = None, device="cpu"):
    """Table [max_pos, rot] = [cos(rot/2) | sin(rot/2)] in float32."""
    half = rot // 2
    inv_freq = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64, device=device) / half))
    mag = 1.0
    if scaling:
        kind = scaling.get("type", scaling.get("rope_type", "linear"))
        factor = float(scaling.get("factor", 1.0))
        if kind == "linear":
            inv_freq = inv_freq / factor
        elif kind == "factors":           # per-frequency divisors (a checkpoint's ``rope_freqs`` tensor)
            inv_freq = inv_freq / torch.tensor(scaling["factors"], dtype=torch.float64, device=device)
        elif kind == "llama3":
            low = float(scaling.get("low_freq_factor", 1.0))
            high = float(scaling.get("high_freq_factor", 4.0))
            orig = float(scaling.get("original_max_position_embeddings", 8192))
            wavelen = 2 * math.pi / inv_freq
            smooth = (orig / wavelen - low) / (high - low)
            scaled = torch.where(wavelen > orig / low, inv_freq / factor, inv_freq)
            mid = (1 - smooth) * inv_freq / factor + smooth * inv_freq
            is_mid = (wavelen <= orig / low) & (wavelen >= orig / high)
            inv_freq = torch.where(is_mid, mid, scaled)
        elif kind == "yarn":
            # NTK-by-parts: high-frequency pairs keep their wavelength, low-frequency pairs are interpolated by
            # ``factor``, a linear ramp between the pairs that turn beta_fast and beta_slow times over the original
            # context; cos and sin carry the attention factor (0.1 ln(factor) + 1 unless the checkpoint gives one,
            # or the ratio of its two mscale terms)
            orig = float(scaling.get("original_max_position_embeddings") or max_pos)
            fast, slow = float(scaling.get("beta_fast") or 32.0), float(scaling.get("beta_slow") or 1.0)

            def corr(n_rot):
                return rot * math.log(orig / (n_rot * 2 * math.pi)) / (2 * math.log(theta))

            lo, hi = corr(fast), corr(slow)
            if scaling.get("truncate", True):
                lo, hi = math.floor(lo), math.ceil(hi)
            lo, hi = max(lo, 0), min(hi, rot - 1)
            if lo == hi:
                hi += 0.001
            ramp = ((torch.arange(half, dtype=torch.float64, device=device) - lo) / (hi - lo)).clamp(0, 1)
            inv_freq = inv_freq / factor * ramp + inv_freq * (1 - ramp)
            mag = yarn_attention_factor(scaling)
    pos = torch.arange(max_pos, dtype=torch.float64, device=device)
    ang = pos[:, None] * inv_freq[None, :]
    return (torch.cat([ang.cos(), ang.sin()], dim=-1) * mag).float()


def yarn_mscale(factor: float, m: float = 1.0) -> float:
    return 1.0 if factor <= 1 else 0.1 * m * math.log(factor) + 1.0


def yarn_attention_factor(scaling: dict) -> float:
    """What YaRN multiplies cos and sin with (so attention scores grow by its square)."""
    if scaling.get("attention_factor") is not None:
        return float(scaling["attention_factor"])
    factor = float(scaling.get("factor", 1.0))
    m, m_all = scaling.get("mscale"), scaling.get("mscale_all_dim")
    if m and m_all:
        return yarn_mscale(factor, float(m)) / yarn_mscale(factor, float(m_all))
    return yarn_mscale(factor)


def apply_rope(x, cos_sin, positions, rot: int):
    """x: [T, H, D]; rotate-half pairing (i, i + rot/2) over the first ``rot`` dims."""
    if rot <= 0:
        return x
    half = rot // 2
    cs = cos_sin[positions.long()]
    c, s = cs[:, None, :half], cs[:, None, half:rot]
    xf = x.float()
    a, b = xf[..., :half], xf[..., half:rot]
    out = xf.clone()
    out[..., :half] = a * c - b * s
    out[..., half:rot] = b * c + a * s
    return out.to(x.dtype)


def head_rmsnorm(x, w, eps, w_offset=0.0):
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * inv * (w.float() + w_offset)).to(x.dtype)


def qk_norm_rope_append(qkv, n_q, n_kv, d, q_norm_w, k_norm_w, eps, w_offset, cos_sin, rot, positions, slots,
                        k_cache, v_cache, gated_q: bool = False):
    """Splits the fused projection, norms + ropes q and k, appends k, v to the paged cache in place.

    With ``gated_q`` the q block is laid out per head as [q(d) | gate(d)]. Returns (q [T, n_q, d], gate or None).
    """
    T = qkv.shape[0]
    qw = n_q * d * (2 if gated_q else 1)
    qpart = qkv[:, :qw].reshape(T, n_q, -1)
    gate = qpart[..., d:] if gated_q else None
    q = qpart[..., :d]
    k = qkv[:, qw:qw + n_kv * d].reshape(T, n_kv, d)
    v = qkv[:, qw + n_kv * d:qw + 2 * n_kv * d].reshape(T, n_kv, d)
    if q_norm_w is not None:
        q = head_rmsnorm(q, q_norm_w, eps, w_offset)
    if k_norm_w is not None:
        k = head_rmsnorm(k, k_norm_w, eps, w_offset)
    q = apply_rope(q, cos_sin, positions, rot)
    k = apply_rope(k, cos_sin, positions, rot)
    page = k_cache.shape[1]
    valid = slots >= 0
    sl = slots[valid].long()
    k_cache.view(-1, n_kv, d)[sl] = k[valid].to(k_cache.dtype)
    v_cache.view(-1, n_kv, d)[sl] = v[valid].to(v_cache.dtype)
    _ = page
    return q.contiguous(), gate


def _gather_kv(cache, table_row, n_tokens):
    page = cache.shape[1]
    n_blocks = (n_tokens + page - 1) // page
    blocks = table_row[:n_blocks].long()
    return cache[blocks].reshape(-1, cache.shape[2], cache.shape[3])[:n_tokens]


def paged_attention(q, k_cache, v_cache, block_table, ctx_lens, cu_q, scale, window: int = 0, causal: bool = True,
                    sinks=None, softcap: float = 0.0):
    """Varlen paged attention. q: [T, Hq, D]; sequence i owns query rows cu_q[i]:cu_q[i+1], which are the
    LAST rows of its ctx_lens[i] cached tokens. Returns [T, Hq, D]."""
    T, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    G = Hq // Hkv
    out = torch.zeros_like(q)
    for i in range(len(ctx_lens)):
        q0, q1 = int(cu_q[i]), int(cu_q[i + 1])
        if q1 <= q0:
            continue
        ctx = int(ctx_lens[i])
        k = _gather_kv(k_cache, block_table[i], ctx).float()
        v = _gather_kv(v_cache, block_table[i], ctx).float()
        qi = q[q0:q1].float()
        k = k.repeat_interleave(G, dim=1)
        v = v.repeat_interleave(G, dim=1)
        s = torch.einsum("qhd,khd->hqk", qi, k) * scale
        if softcap > 0:
            s = torch.tanh(s / softcap) * softcap
        qpos = torch.arange(ctx - (q1 - q0), ctx, device=q.device)[:, None]
        kpos = torch.arange(ctx, device=q.device)[None, :]
        mask = torch.ones(q1 - q0, ctx, dtype=torch.bool, device=q.device)
        if causal:
            mask &= kpos <= qpos
        if window > 0:
            mask &= kpos > qpos - window
        s = s.masked_fill(~mask[None], float("-inf"))
        if sinks is not None:
            s = torch.cat([s, sinks.float().view(Hq, 1, 1).expand(Hq, q1 - q0, 1)], dim=-1)
            p = torch.softmax(s, dim=-1)[..., :-1]
        else:
            p = torch.softmax(s, dim=-1)
        p = torch.nan_to_num(p)
        out[q0:q1] = torch.einsum("hqk,khd->qhd", p, v).to(q.dtype)
    return out


def router_topk(logits, k: int, mode: str = "softmax", renorm: bool = True, route_scale: float = 1.0, bias=None,
                n_group: int = 1, topk_group: int = 1):
    """Returns (ids [T, k] int32, weights [T, k] float32); ties go to the lower expert id."""
    lf = logits.float()
    T, E = lf.shape
    if mode == "softmax":
        scores = torch.softmax(lf, dim=-1)
        sel = scores.clone()
    else:
        scores = torch.sigmoid(lf)
        sel = scores + (bias.float() if bias is not None else 0.0)
        if n_group > 1 and topk_group < n_group:
            g = sel.view(T, n_group, E // n_group)
            gscore = g.topk(min(2, g.shape[-1]), dim=-1).values.sum(-1)
            order = torch.sort(gscore, dim=-1, descending=True, stable=True).indices[:, :topk_group]
            keep = torch.zeros(T, n_group, dtype=torch.bool, device=lf.device)
            keep.scatter_(1, order, True)
            sel = g.masked_fill(~keep[:, :, None], float("-inf")).reshape(T, E)
    order = torch.sort(sel, dim=-1, descending=True, stable=True).indices[:, :k]
    w = scores.gather(1, order)
    if renorm:
        w = w / w.sum(-1, keepdim=True).clamp_min(6.1e-5)
    return order.int(), (w * route_scale).float()


def moe_experts(x, ids, wts, w_gate_up, w_down, n_ff: int, act: str = "silu", e_lo: int = 0, e_hi: Optional[int] = None):
    """Routed expert FFN. w_gate_up: [E, 2*n_ff, H] ([gate | up] rows), w_down: [E, H, n_ff].
    Only experts in [e_lo, e_hi) contribute (expert parallel shards). Returns float32 [T, H]."""
    T, H = x.shape
    E = w_gate_up.shape[0]
    e_hi = E + e_lo if e_hi is None else e_hi
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    xf = x.float()
    for e in range(e_lo, e_hi):
        hit = ids == e
        if not bool(hit.any()):
            continue
        tok, choice = hit.nonzero(as_tuple=True)
        le = e - e_lo
        h = xf[tok] @ w_gate_up[le].float().t()
        if h.shape[1] == n_ff:            # un-gated experts (squared ReLU): one up projection
            h = activation(h, act).to(x.dtype).float()
        else:
            h = (activation(h[:, :n_ff], act) * h[:, n_ff:]).to(x.dtype).float()
        y = (h @ w_down[le].float().t()) * wts[tok, choice][:, None]
        out.index_add_(0, tok, y.to(x.dtype).float())
    return out


def argmax(logits):
    return torch.argmax(logits.float(), dim=-1).int()


def causal_conv1d_silu(x, w, bias, conv_state, cu_seq, slots, write_state: bool = True):
    """x: [T, C]; w: [C, KC]; conv_state: [slots, C, KC-1] float32 (oldest first)."""
    out = torch.empty_like(x)
    KC = w.shape[1]
    for i in range(len(slots)):
        t0, t1 = int(cu_seq[i]), int(cu_seq[i + 1])
        if t1 <= t0:
            continue
        s = int(slots[i])
        hist = conv_state[s].float().t()  # [KC-1, C]
        seq = torch.cat([hist, x[t0:t1].float()], dim=0)
        win = seq.unfold(0, KC, 1)  # [n, C, KC]
        y = (win * w.float()[None]).sum(-1)
        if bias is not None:
            y = y + bias.float()
        out[t0:t1] = F.silu(y).to(x.dtype)
        if write_state:
            conv_state[s] = seq[-(KC - 1):].t().to(conv_state.dtype)
    return out


def gdn_gates(a, b, A, dt_bias):
    g = A.float() * F.softplus(a.float() + dt_bias.float())
    return g, torch.sigmoid(b.float())


def gdn_recurrent(qkv, g, beta, state, cu_seq, slots, n_k, n_v, dk, dv, tiled_heads: bool, scale: float,
                  l2_eps: float = 1e-6, write_state: bool = True):
    """Gated delta rule, token by token. qkv: [T, 2*n_k*dk + n_v*dv]; state: [slots, n_v, dk, dv] float32."""
    T = qkv.shape[0]
    out = torch.zeros(T, n_v, dv, dtype=qkv.dtype, device=qkv.device)
    q_all = qkv[:, :n_k * dk].float().view(T, n_k, dk)
    k_all = qkv[:, n_k * dk:2 * n_k * dk].float().view(T, n_k, dk)
    v_all = qkv[:, 2 * n_k * dk:].float().view(T, n_v, dv)
    q_all = q_all * torch.rsqrt(q_all.pow(2).sum(-1, keepdim=True) + l2_eps) * scale
    k_all = k_all * torch.rsqrt(k_all.pow(2).sum(-1, keepdim=True) + l2_eps)
    heads = torch.arange(n_v, device=qkv.device)
    kh = heads % n_k if tiled_heads else heads // (n_v // n_k)
    for i in range(len(slots)):
        t0, t1 = int(cu_seq[i]), int(cu_seq[i + 1])
        s = int(slots[i])
        S = state[s].float().clone()  # [n_v, dk, dv]
        for t in range(t0, t1):
            q, k, v = q_all[t, kh], k_all[t, kh], v_all[t]
            gt = torch.exp(g[t].float())[:, None]
            bt = beta[t].float()[:, None]
            kv = torch.einsum("hkv,hk->hv", S, k)
            delta = (v - gt * kv) * bt
            S = gt[:, :, None] * S + k[:, :, None] * delta[:, None, :]
            out[t] = torch.einsum("hkv,hk->hv", S, q).to(out.dtype)
        if write_state:
            state[s] = S.to(state.dtype)
    return out


def gated_rmsnorm(o, z, w, eps: float, act: str = "silu"):
    """o, z: [T, H, D]; w: [D]."""
    of = o.float()
    y = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    zf = z.float()
    return (y * (F.silu(zf) if act == "silu" else torch.sigmoid(zf))).to(o.dtype)


def sample(logits, temperature, top_k, top_p, min_p, generator=None):
    """Host-order sampling for one row: temperature -> min-p -> top-k -> top-p -> draw."""
    lf = logits.float()
    if temperature <= 0:
        return int(torch.argmax(lf))
    p = torch.softmax(lf / temperature, dim=-1)
    if min_p and min_p > 0:
        p = torch.where(p >= min_p * p.max(), p, torch.zeros_like(p))
    if top_k and 0 < top_k < p.numel():
        kth = torch.topk(p, top_k).values[-1]
        p = torch.where(p >= kth, p, torch.zeros_like(p))
    if top_p is not None and top_p < 1.0:
        sp, si = torch.sort(p, descending=True)
        csum = torch.cumsum(sp, 0) / sp.sum()
        keep = (csum - sp / sp.sum()) < top_p
        mask = torch.zeros_like(p, dtype=torch.bool)
        mask[si[keep]] = True
        p = torch.where(mask, p, torch.zeros_like(p))
    p = p / p.sum()
    return int(torch.multinomial(p, 1, generator=generator))
