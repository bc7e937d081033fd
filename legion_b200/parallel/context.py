"""Parallel context: how one rank's partial results become the next sub-layer's input.

The decoder never calls a collective itself; it hands the (possibly rank-partial) output of a
sub-layer to ``ParallelCtx.reduce_norm`` together with the residual stream and the next norm weight.
  * world 1 ............... fused residual-add + RMSNorm kernel.
  * ``comm="nccl"`` ....... baseline: ``dist.all_reduce`` (NCCL on GPUs, gloo on CPU ranks) followed by
                            the residual-add + RMSNorm kernel.
  * ``comm="fused"`` ...... the o-proj / down-proj GEMM epilogue writes its partial tile straight into
                            this rank's symmetric buffer; one kernel then signals the peers, waits for
                            theirs, sums the partials in rank order over NVLink peer loads, adds the
                            residual and applies the norm (``csrc/comm.cu``). Large steps use the
                            two-shot form (reduce-scatter + all-gather kernels).
Reference counterparts: ``src/tp_net/op.rs:26-60`` (all_reduce, all_reduce_add_norm),
``src/tp_net/micro/send_gemm.rs`` (GEMM writes into the send buffer), ``src/model/core/tp_ep.rs`` (EP by
summing partial MoE outputs), ``src/model/core/tp.rs:110`` (Megatron split).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops


class PendingLinear:
    """A projection whose result is a rank-partial sum: kept unevaluated so that the reduction that follows can
    run it and the all-reduce as one kernel (``SymmComm.linear_reduce_norm``)."""
    __slots__ = ("x", "w")

    def __init__(self, x, w):
        self.x, self.w = x, w


class ParallelCtx:
    def __init__(self, rank: int = 0, world: int = 1, group=None, expert_parallel: bool = False, comm: str = "nccl",
                 symm=None, gemm_tail: bool = False):
        self.rank, self.world, self.group = rank, world, group
        self.tp = world
        self.ep = expert_parallel and world > 1
        self.comm = comm if world > 1 else "none"
        self.symm = symm  # parallel.symm.SymmComm when comm == "fused"
        # run o-proj / down-proj and their all-reduce as ONE kernel (``SymmComm.linear_reduce_norm``). Off by
        # default: at decode sizes the extra grid-wide arrive inside the GEMM costs more than the second launch
        # (8.42 vs 8.08 ms per step at TP=2 on the 30B-A3B shape).
        self.gemm_tail = gemm_tail
        self.stats = {"all_reduce": 0, "bytes": 0}

    @classmethod
    def single(cls) -> "ParallelCtx":
        return cls()

    def expert_range(self, n_expert: int):
        if not self.ep:
            return 0, n_expert
        per = n_expert // self.world
        return self.rank * per, (self.rank + 1) * per

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return x
        self.stats["all_reduce"] += 1
        self.stats["bytes"] += x.numel() * x.element_size()
        if self.comm == "fused" and x.is_cuda and x.shape[0] <= self.symm.max_rows:
            return self.symm.all_reduce(x)
        import torch.distributed as dist
        if x.dtype == torch.bfloat16 and not x.is_cuda:
            y = x.float()
            dist.all_reduce(y, group=self.group)
            return y.to(x.dtype)
        dist.all_reduce(x, group=self.group)
        return x

    def partial_out(self, rows: int, cols: int) -> Optional[torch.Tensor]:
        """Where the GEMM before a reduction should write: a slice of the symmetric buffer (fused path)."""
        if self.comm == "fused" and self.symm is not None:
            return self.symm.next_partial(rows, cols)
        return None

    def defer_linear(self, x, w, lazy: bool = False):
        """x @ w^T whose output is rank-partial. With the fused communicator on a GPU the GEMM is deferred to the
        next ``reduce_norm`` (GEMM + all-reduce + residual + norm in one launch); otherwise it runs now, writing
        into the symmetric slot when there is one. ``lazy``: on a single rank the projection is also kept
        unevaluated, so that its consumer can run it with the residual added in the GEMM epilogue."""
        rows, cols = x.shape[0], w.shape[0]
        if lazy and self.world == 1:
            return PendingLinear(x, w)
        if (self.world > 1 and self.comm == "fused" and self.symm is not None and x.is_cuda and self.gemm_tail
                and self.symm.fits_gemm_tail(rows, cols)):
            return PendingLinear(x, w)
        return ops.linear(x, w, out=self.partial_out(rows, cols))

    def _materialize(self, cur):
        if isinstance(cur, ops.sm100.PendingCombine):
            return cur.materialize(self.partial_out(cur.T, cur.H))
        if isinstance(cur, PendingLinear):
            return ops.linear(cur.x, cur.w, out=self.partial_out(cur.x.shape[0], cur.w.shape[0]))
        return cur

    def end_step(self):
        if self.comm == "fused" and self.symm is not None:
            self.symm.end_step()

    def reduce_norm_quant(self, cur, res, w, eps, w_offset):
        """``reduce_norm`` of a decode-sized step whose consumer is an NVFP4 expert block: returns (normed, hidden,
        encoded rows). With the fused communicator the encoding comes out of the reduction launch itself."""
        if isinstance(cur, ops.sm100.PendingCombine) and res is not None and self._fused_combine_ok(cur):
            self.stats["all_reduce"] += 1
            self.stats["bytes"] += cur.T * cur.H * 2
            return self.symm.all_reduce_add_norm(self.symm.next_partial(cur.T, cur.H), res, w, eps, w_offset, quant=True,
                                                 combine=cur)
        cur = self._materialize(cur)
        if (self.world > 1 and self.comm == "fused" and cur is not None and res is not None and cur.is_cuda
                and self.symm.owns(cur) and cur.shape[1] % 256 == 0):
            self.stats["all_reduce"] += 1
            self.stats["bytes"] += cur.numel() * cur.element_size()
            return self.symm.all_reduce_add_norm(cur, res, w, eps, w_offset, quant=True)
        normed, hidden = self.reduce_norm(cur, res, w, eps, w_offset)
        return normed, hidden, ops.sm100.nv4_quant_act(normed, key="ffn_in")

    def reduce_norm(self, cur, res, w, eps, w_offset):
        """hidden = reduce(cur) + res; returns (rmsnorm(hidden) * w, hidden).

        ``cur`` is None when the previous kernel already produced the full stream in ``res``;
        ``res`` is None right after the embedding (``cur`` is then complete, not partial)."""
        if cur is None:
            normed, _ = ops.rmsnorm(res, w, eps, w_offset)
            return normed, res
        if isinstance(cur, ops.sm100.PendingCombine):
            if res is not None and self._fused_combine_ok(cur):
                self.stats["all_reduce"] += 1
                self.stats["bytes"] += cur.T * cur.H * 2
                return self.symm.all_reduce_add_norm(self.symm.next_partial(cur.T, cur.H), res, w, eps, w_offset,
                                                     combine=cur)
            cur = self._materialize(cur)
        if isinstance(cur, PendingLinear) and self.world == 1:
            hidden = ops.linear(cur.x, cur.w, residual=res)
            normed, _ = ops.rmsnorm(hidden, w, eps, w_offset)
            return normed, hidden
        if isinstance(cur, PendingLinear):
            if res is not None:
                self.stats["all_reduce"] += 1
                self.stats["bytes"] += cur.x.shape[0] * cur.w.shape[0] * 2
                return self.symm.linear_reduce_norm(cur.x, cur.w, res, w, eps, w_offset)
            cur = self._materialize(cur)
        if res is None:
            normed, _ = ops.rmsnorm(cur, w, eps, w_offset)
            return normed, cur
        if self.world > 1:
            if self.comm == "fused" and cur.is_cuda and self.symm.owns(cur):
                self.stats["all_reduce"] += 1
                self.stats["bytes"] += cur.numel() * cur.element_size()
                return self.symm.all_reduce_add_norm(cur, res, w, eps, w_offset)
            cur = self.all_reduce(cur)
        return ops.rmsnorm(cur, w, eps, w_offset, residual=res)

    def _fused_combine_ok(self, pc) -> bool:
        return (self.world > 1 and self.comm == "fused" and self.symm is not None and pc.T <= self.symm.LL_ROWS
                and pc.H == self.symm.hidden and bool(ops.sm100.TUNE.get("ar_ll", 1)))

    def full_hidden(self, cur, res):
        if isinstance(cur, PendingLinear) and self.world == 1 and res is not None:
            return ops.linear(cur.x, cur.w, residual=res)
        cur = self._materialize(cur)
        if cur is None:
            return res
        if res is None:
            return cur
        if self.world > 1:
            cur = self.all_reduce(cur)
        return (cur.float() + res.float()).to(res.dtype)

    def moe(self, x, ids, wts, w_gate_up, w_down, n_ff, act, e_lo, shared, shared_gate, residual, norm=None, routing=None):
        """Routed experts of this rank: all experts with their FFN rows split (TP) or whole local
        experts (EP). Either way the result is a partial sum that the next ``reduce_norm`` completes."""
        defer = (x.is_cuda and self.world > 1 and self.comm == "fused" and self.symm is not None and residual is None
                 and norm is None and x.shape[0] <= self.symm.LL_ROWS and bool(ops.sm100.TUNE.get("ar_combine", 1)))
        return ops.moe_experts(x, ids, wts, w_gate_up, w_down, n_ff, act, e_lo, shared, shared_gate, residual,
                               out=self.partial_out(x.shape[0], x.shape[1]) if x.is_cuda else None, norm=norm,
                               routing=routing, defer_combine=defer)


class DpEpCtx(ParallelCtx):
    """Data-parallel attention with expert parallelism: every rank holds the attention / dense / shared-expert
    weights whole and ``E / world`` routed experts, runs attention only for the sequences it owns, and meets the
    other ranks inside each MoE layer, where tokens travel to their experts' owners and the results come back
    (``parallel.ep.EpDispatcher`` on GPUs: dispatch and combine are peer stores fused into the grouped GEMM
    pipeline; on CPU ranks the same exchange is an all-gather of the padded tokens, local experts over all of
    them, and a sum). To the decoder it looks like a single rank: no layer output is a partial sum.

    Reference counterpart: none (the reference mirrors tokens on every rank, ``src/model/core/tp_ep.rs:8-11``)."""

    def __init__(self, rank: int, world: int, group, dispatcher=None):
        super().__init__(0, 1)
        self.dp_rank, self.dp_world, self.dp_group = rank, world, group
        self.dispatcher = dispatcher
        self.ep = world > 1

    def expert_range(self, n_expert: int):
        per = n_expert // self.dp_world
        return self.dp_rank * per, (self.dp_rank + 1) * per

    def moe(self, x, ids, wts, w_gate_up, w_down, n_ff, act, e_lo, shared, shared_gate, residual, norm=None,
            routing=None):
        if x.is_cuda:
            if act != "silu":
                raise NotImplementedError("the expert-parallel exchange implements SwiGLU experts")
            y = self.dispatcher.forward(x, ids, wts, w_gate_up, w_down, shared, shared_gate, residual)
        else:
            y = self._moe_gathered(x, ids, wts, w_gate_up, w_down, n_ff, act, e_lo)
            if shared is not None:
                sh = shared.float()
                if shared_gate is not None:
                    sh = sh * torch.sigmoid(shared_gate.float())[:, None]
                y = y + sh
            if residual is not None:
                y = y + residual.float()
            y = y.to(x.dtype)
        if norm is None:
            return y
        normed, _ = ops.rmsnorm(y, norm[0], norm[1], norm[2])
        return y, normed

    def _moe_gathered(self, x, ids, wts, w_gate_up, w_down, n_ff, act, e_lo):
        """CPU ranks: all tokens to all ranks, local experts over all of them, sum, keep the own rows."""
        import torch.distributed as dist
        W, R, g = self.dp_world, self.dp_rank, self.dp_group
        T = x.shape[0]
        sizes = [torch.zeros(1, dtype=torch.int64) for _ in range(W)]
        dist.all_gather(sizes, torch.tensor([T], dtype=torch.int64), group=g)
        sizes = [int(t.item()) for t in sizes]
        M = max(sizes)

        def gather(t, fill=0):
            pad = torch.full((M,) + tuple(t.shape[1:]), fill, dtype=t.dtype)
            pad[:T] = t
            outs = [torch.empty_like(pad) for _ in range(W)]
            dist.all_gather(outs, pad, group=g)
            return torch.cat([o[:n] for o, n in zip(outs, sizes)], 0)

        xa, ia, wa = gather(x.float()), gather(ids, -1), gather(wts.float())
        ya = ops.reference.moe_experts(xa.to(x.dtype), ia, wa, w_gate_up, w_down, n_ff, act, e_lo,
                                       e_lo + w_gate_up.shape[0])
        dist.all_reduce(ya, group=g)
        off = sum(sizes[:R])
        return ya[off:off + T]
