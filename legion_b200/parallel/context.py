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
        if isinstance(cur, PendingLinear):
            return ops.linear(cur.x, cur.w, out=self.partial_out(cur.x.shape[0], cur.w.shape[0]))
        return cur

    def end_step(self):
        if self.comm == "fused" and self.symm is not None:
            self.symm.end_step()

    def reduce_norm(self, cur, res, w, eps, w_offset):
        """hidden = reduce(cur) + res; returns (rmsnorm(hidden) * w, hidden).

        ``cur`` is None when the previous kernel already produced the full stream in ``res``;
        ``res`` is None right after the embedding (``cur`` is then complete, not partial)."""
        if cur is None:
            normed, _ = ops.rmsnorm(res, w, eps, w_offset)
            return normed, res
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
        return ops.moe_experts(x, ids, wts, w_gate_up, w_down, n_ff, act, e_lo, shared, shared_gate, residual,
                               out=self.partial_out(x.shape[0], x.shape[1]) if x.is_cuda else None, norm=norm,
                               routing=routing)
