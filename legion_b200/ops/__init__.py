"""Ops: one function per kernel family.

CUDA tensors run the hand-written sm_100a kernels (``ops.sm100``; the extension is required, there is
no eager fallback on a GPU). CPU tensors run the float32 PyTorch reference (``ops.reference``), which
is both the test oracle and the back-end of the CPU engine used by the scheduler / cache / speculative
decoding tests.
"""
from __future__ import annotations

import torch

from . import reference as _ref
from . import sm100 as _sm

reference = _ref
sm100 = _sm


def _cuda(t) -> bool:
    return t.is_cuda


def linear(x, w, residual=None, out_dtype=None, out=None):
    if _cuda(x):
        return _sm.linear(x, w, residual=residual, out=out, out_dtype=out_dtype or torch.bfloat16)
    y = _ref.linear(x, w, residual=residual, out_dtype=out_dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def gate_up_act(x, w_gate_up, n_ff, act="silu"):
    if _cuda(x):
        if act == "silu":
            return _sm.gate_up_act(x, w_gate_up, n_ff)
        h = _sm.linear(x, w_gate_up)
        out = torch.empty(x.shape[0], n_ff, dtype=torch.bfloat16, device=x.device)
        _sm.ext().glu(h, out, n_ff, {"gelu_tanh": 1, "relu2": 2}[act])
        return out
    return _ref.gate_up_act(x, w_gate_up, n_ff, act)


def rmsnorm(x, w, eps, w_offset=0.0, residual=None):
    """Returns (normed, summed)."""
    if _cuda(x):
        return _sm.rmsnorm(x, w, eps, w_offset, residual)
    return _ref.rmsnorm(x, w, eps, w_offset, residual)


def qk_norm_rope_append(qkv, n_q, n_kv, d, q_norm_w, k_norm_w, eps, w_offset, cos_sin, rot, positions, slots, k_cache,
                        v_cache, gated_q=False):
    """Returns (q [T, n_q, d], gate handle). On CUDA the gate stays inside ``qkv`` (handle = qkv)."""
    if _cuda(qkv):
        q = _sm.qk_norm_rope_append(qkv, n_q, n_kv, d, q_norm_w, k_norm_w, eps, w_offset, cos_sin, rot, positions,
                                    slots, k_cache, v_cache, gated_q)
        return q, (qkv if gated_q else None)
    return _ref.qk_norm_rope_append(qkv, n_q, n_kv, d, q_norm_w, k_norm_w, eps, w_offset, cos_sin, rot, positions,
                                    slots, k_cache, v_cache, gated_q)


def apply_output_gate(attn, gate, n_q, d):
    """attn [T, n_q, d] * sigmoid(gate)."""
    if _cuda(attn):
        return _sm.sigmoid_gate(attn, gate, n_q, d)
    return (attn.float() * torch.sigmoid(gate.float())).to(attn.dtype)


def paged_attention(q, k_cache, v_cache, block_table, ctx_lens, cu_q, max_q_len, scale, window=0, causal=True,
                    decode_splits=None, max_ctx=None):
    """Varlen paged attention; ``max_q_len == 1`` selects the flash-decoding kernel on CUDA."""
    if _cuda(q):
        if max_q_len == 1 and causal:
            return _sm.paged_decode(q, k_cache, v_cache, block_table, ctx_lens, scale, window, decode_splits, max_ctx)
        return _sm.prefill_attn(q, k_cache, v_cache, cu_q, ctx_lens, block_table, max_q_len, scale, window, causal)
    return _ref.paged_attention(q, k_cache, v_cache, block_table, ctx_lens, cu_q, scale, window, causal)


def router_topk(logits, k, mode="softmax", renorm=True, route_scale=1.0, bias=None, n_group=1, topk_group=1):
    if _cuda(logits):
        return _sm.router_topk(logits, k, mode, renorm, route_scale, bias, n_group, topk_group)
    return _ref.router_topk(logits, k, mode, renorm, route_scale, bias, n_group, topk_group)


def router(x, w_router, k, mode="softmax", renorm=True, route_scale=1.0, bias=None, n_group=1, topk_group=1,
           e_lo=0, n_local=None, norm=None, **gpu_kw):
    """Router projection + top-k. Returns an object that unpacks as ``ids, wts`` ([T, k] int32 / float32); on the
    GPU it may also carry the dense routing tables of a decode-sized step for the experts
    [e_lo, e_lo + n_local) of this rank (pass it on as ``routing=``). With ``norm=(weight, eps, w_offset)`` ``x`` is
    the raw residual stream: the RMSNorm runs first (inside the routing launch for decode-sized steps on the GPU)
    and the result's ``x_normed`` is the normalised input for the experts."""
    if _cuda(x):
        return _sm.router(x, w_router, k, mode, renorm, route_scale, bias, n_group, topk_group, norm, e_lo, n_local,
                          **gpu_kw)
    xn = None
    if norm is not None:
        xn, _ = _ref.rmsnorm(x, norm[0], norm[1], norm[2])
    logits = _ref.linear(x if xn is None else xn, w_router, out_dtype=torch.float32)
    ids, wts = _ref.router_topk(logits, k, mode, renorm, route_scale, bias, n_group, topk_group)
    return _sm.Routing(ids, wts, None, xn)


def _moe_experts_ungated(x, ids, wts, w_up, w_down, e_lo, shared, shared_gate, residual, norm, act="relu2", n_ff=None):
    """Experts the grouped kernels do not cover (un-gated squared ReLU, GELU-gated) on a GPU by tensor operations:
    pairs sorted by expert, one batched product per weight over padded per-expert groups."""
    T, H = x.shape
    E = w_up.shape[0]
    k = ids.shape[1]
    flat = ids.reshape(-1).long() - e_lo
    mine = (flat >= 0) & (flat < E)
    tok = torch.arange(T, device=x.device).repeat_interleave(k)
    key = torch.where(mine, flat, torch.full_like(flat, E))
    order = torch.argsort(key, stable=True)
    counts = torch.zeros(E + 1, dtype=torch.int64, device=x.device).scatter_add_(0, key, torch.ones_like(key))[:E]
    cap = T * k if T * k <= 64 else int(counts.max().item())          # small steps: no host read
    cap = max(cap, 1)
    starts = torch.cumsum(counts, 0) - counts
    pos = torch.arange(cap, device=x.device)[None, :]                 # [1, cap]
    src = (starts[:, None] + pos).clamp(max=T * k - 1)                # [E, cap] index into the sorted pairs
    live = pos < counts[:, None]
    pair = order[src]                                                 # [E, cap] pair index
    xg = x[tok[pair]] * live[..., None].to(x.dtype)                   # [E, cap, H]
    h = torch.bmm(xg, w_up.transpose(1, 2))
    if n_ff is not None and h.shape[-1] == 2 * n_ff:       # gated: [gate | up]
        h = (_ref.activation(h[..., :n_ff].float(), act) * h[..., n_ff:].float()).to(x.dtype)
    else:
        h = _ref.activation(h.float(), act).to(x.dtype)
    y = torch.bmm(h, w_down.transpose(1, 2)).float()                  # [E, cap, H]
    y = y * (wts.reshape(-1)[pair] * live).unsqueeze(-1)
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    out.index_add_(0, tok[pair].reshape(-1), y.reshape(-1, H))
    if shared is not None:
        s = shared.float()
        if shared_gate is not None:
            s = s * torch.sigmoid(shared_gate.float())[:, None]
        out = out + s
    if residual is not None:
        out = out + residual.float()
    out = out.to(x.dtype)
    if norm is None:
        return out
    return out, rmsnorm(out, norm[0], norm[1], norm[2])[0]


def moe_experts(x, ids, wts, w_gate_up, w_down, n_ff, act="silu", e_lo=0, shared=None, shared_gate=None,
                residual=None, out=None, norm=None, routing=None, defer_combine=False):
    """Routed experts (+ optional shared-expert output with sigmoid gate logits, + residual). Returns [T, H];
    with ``norm=(weight, eps, w_offset)`` returns (out, rmsnorm(out)): on the GPU the norm rides on the combine."""
    if _cuda(x) and act != "silu":
        if act not in ("relu2", "gelu_tanh") or not isinstance(w_gate_up, torch.Tensor):
            raise NotImplementedError("the grouped expert kernels implement SwiGLU experts (squared-ReLU and GELU "
                                      "experts run through tensor operations)")
        # un-gated squared-ReLU experts (Nemotron-H) and GELU-gated experts (Gemma 4): no grouped kernel of their own
        # yet; the per-expert products run as tensor operations over the tokens of each expert, on the device,
        # without a host round trip per expert
        return _moe_experts_ungated(x, ids, wts, w_gate_up, w_down, e_lo, shared, shared_gate, residual, norm, act, n_ff)
    if _cuda(x):
        return _sm.moe_experts(x, ids, wts, w_gate_up, w_down, n_ff, e_lo, None, shared, shared_gate, residual, out,
                               norm, routing if isinstance(routing, _sm.Routing) else None,
                               defer_combine=defer_combine)
    y = _ref.moe_experts(x, ids, wts, w_gate_up, w_down, n_ff, act, e_lo, e_lo + w_gate_up.shape[0])
    if shared is not None:
        s = shared.float()
        if shared_gate is not None:
            s = s * torch.sigmoid(shared_gate.float())[:, None]
        y = y + s
    if residual is not None:
        y = y + residual.float()
    y = y.to(x.dtype)
    if norm is None:
        return y
    return y, _ref.rmsnorm(y, norm[0], norm[1], norm[2])[0]


def argmax(logits):
    if _cuda(logits):
        return _sm.argmax(logits)
    return _ref.argmax(logits)


def embed(ids, table):
    if _cuda(table):
        return _sm.embed(ids.int(), table)
    return table[ids.long()]


def causal_conv1d_silu(x, w, bias, conv_state, cu_seq, slots, write_state=True, max_len=None):
    if _cuda(x):
        return _sm.causal_conv1d_silu(x, w, bias, conv_state, cu_seq, slots, write_state, max_len=max_len)
    return _ref.causal_conv1d_silu(x, w, bias, conv_state, cu_seq, slots, write_state)


def gdn_gates(a, b, A, dt_bias):
    if _cuda(a):
        return _sm.gdn_gates(a, b, A, dt_bias)
    return _ref.gdn_gates(a, b, A, dt_bias)


def gdn_recurrent(qkv, g, beta, state, cu_seq, slots, n_k, n_v, dk, dv, tiled_heads, scale, l2_eps=1e-6,
                  write_state=True, cu_host=None):
    if _cuda(qkv):
        return _sm.gdn_recurrent(qkv, g, beta, state, cu_seq, slots, n_k, n_v, dk, dv, tiled_heads, scale, l2_eps,
                                 write_state, cu_host=cu_host)
    return _ref.gdn_recurrent(qkv, g, beta, state, cu_seq, slots, n_k, n_v, dk, dv, tiled_heads, scale, l2_eps,
                              write_state)


def gated_rmsnorm(o, z, w, eps, act="silu"):
    if _cuda(o):
        return _sm.gated_rmsnorm(o, z, w, eps, act)
    return _ref.gated_rmsnorm(o, z.reshape(o.shape), w, eps, act)
