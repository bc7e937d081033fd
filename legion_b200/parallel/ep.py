"""Expert-parallel MoE with token dispatch / result combine fused into the GEMM pipeline.

Each rank keeps its own tokens (data-parallel attention) and ``E / world`` whole experts. One MoE layer is

    plan (all E experts) -> publish counts -> push rows to the owners' receive buffers (peer stores)
      -> wait for all sources -> grouped gate/up GEMM (+SwiGLU) over the receive buffer
      -> grouped down GEMM whose epilogue scales by the routing weight and stores every output row straight
         into the SOURCE rank's pair buffer over NVLink -> flag round -> local combine

so neither all-to-all exists as a separate collective: the dispatch is the plan's gather, the combine is the
down projection's own store. Kernels: ``csrc/ep.cu`` and the ``out_peer`` epilogue of ``csrc/gemm_sm100.cu``.
Every cross-rank wait is bounded; a peer that does not arrive sets the status word (``check``).

The reference has no token all-to-all: it mirrors tokens on every rank and all-reduces the partial outputs
(``src/model/core/tp_ep.rs:8-11``); that form is ``ParallelCtx.moe`` with ``ep=True``.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops.sm100 import MoePlan, Workspace, ext


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class EpError(RuntimeError):
    pass


class EpDispatcher:
    """Symmetric buffers and launch sequence of the expert-parallel MoE layer.

    max_tokens: largest number of tokens one rank brings to a layer. cap_factor scales the receive buffer
    relative to a perfectly balanced routing (``world`` = worst case: every pair of every rank lands here)."""

    def __init__(self, group, rank: int, world: int, device: torch.device, n_expert: int, top_k: int, hidden: int,
                 n_ff: int, max_tokens: int, cap_factor: Optional[float] = None, budget_ns: int = 5_000_000_000):
        from .dist import no_multicast_default
        no_multicast_default()
        import torch.distributed._symmetric_memory as symm_mem
        if n_expert % world:
            raise ValueError("experts must divide evenly over the ranks")
        self.rank, self.world, self.device = rank, world, device
        self.E, self.k, self.H, self.F = n_expert, top_k, hidden, n_ff
        self.per = n_expert // world
        self.max_tokens = max_tokens
        P = max_tokens * top_k
        cap = P * world if cap_factor is None else min(P * world, int(P * cap_factor) + 1)
        self.bn = 32 if cap <= 32 * self.per else (64 if cap <= 64 * self.per else 128)
        self.cap = cap
        self.max_tiles = (cap + self.bn - 1) // self.bn + self.per
        rows = cap + self.bn
        self.off_counts = 0
        self.off_rx = _align(world * n_expert * 4)
        self.off_rsrc = _align(self.off_rx + rows * hidden * 2)
        self.off_rw = _align(self.off_rsrc + rows * 4)
        self.off_y = _align(self.off_rw + rows * 4)
        nbytes = _align(self.off_y + P * hidden * 2)
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.buf, group=group)
        self.buffer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.signal_ptrs = [int(p) for p in self.handle.signal_pad_ptrs]
        self.buf.zero_()
        b = self.buf
        self.recv_x = b[self.off_rx:self.off_rx + rows * hidden * 2].view(torch.bfloat16).view(rows, hidden)
        self.recv_src = b[self.off_rsrc:self.off_rsrc + rows * 4].view(torch.int32)
        self.recv_w = b[self.off_rw:self.off_rw + rows * 4].view(torch.float32)
        self.y_pairs = b[self.off_y:self.off_y + P * hidden * 2].view(torch.bfloat16).view(P, hidden)
        self.y_peer = [p + self.off_y for p in self.buffer_ptrs]
        i32 = dict(dtype=torch.int32, device=device)
        self.plan = MoePlan(max_tokens, top_k, n_expert, self.bn, device)
        self.dest_base = torch.zeros(n_expert, **i32)
        self.recv_counts = torch.zeros(self.per, **i32)
        self.r_offsets = torch.zeros(self.per + 1, **i32)
        self.tile_group = torch.zeros(self.max_tiles, **i32)
        self.tile_tok0 = torch.zeros(self.max_tiles, **i32)
        self.tile_ntok = torch.zeros(self.max_tiles, **i32)
        self.meta = torch.zeros(4, **i32)            # {n_tiles, n_rows (tile scan), rows received, -}
        self.h = torch.zeros(rows, n_ff, dtype=torch.bfloat16, device=device)
        self.seq = torch.zeros(1, **i32)
        self.done = torch.zeros(1, **i32)
        self.status = torch.zeros(1, **i32)
        self.budget_ns = budget_ns
        self._failed: Optional[str] = None
        torch.cuda.synchronize(device)
        import torch.distributed as dist
        dist.barrier(group=group)

    def forward(self, x: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, w_gate_up: torch.Tensor,
                w_down: torch.Tensor, shared=None, shared_gate=None, residual=None, out=None) -> torch.Tensor:
        """x [T, H] bf16 (this rank's tokens), ids/wts [T, k] over the GLOBAL experts; w_gate_up
        [E/world, 2F, H] and w_down [E/world, H, F] are this rank's experts. Returns [T, H] bf16."""
        if self._failed:
            raise EpError(self._failed)
        C = ext()
        T, H = x.shape
        if T > self.max_tokens or H != self.H or ids.shape[1] != self.k:
            raise ValueError("EP layer called outside the shape it was sized for")
        p, P = self.plan, T * self.k
        ws = Workspace.get(x.device)
        peers = (self.buffer_ptrs, self.signal_ptrs, self.rank)
        C.moe_plan(ids, wts, 0, self.E, self.bn, p.counts, p.offsets, p.sorted_token, p.sorted_pair, p.sorted_w,
                   p.tile_group, p.tile_tok0, p.tile_ntok, p.meta)
        C.ep_publish_counts(*peers, p.counts, self.off_counts, self.seq, self.dest_base, self.recv_counts, self.meta,
                            self.cap, self.budget_ns, self.status)
        C.ep_push(*peers, x, p.sorted_token[:P], p.sorted_pair[:P], p.sorted_w[:P], p.offsets, self.dest_base, self.E,
                  self.cap, self.off_rx, self.off_rsrc, self.off_rw, self.seq, self.done)
        C.ep_sync(*peers, 40, False, self.seq, False, self.budget_ns, self.status)          # all sources pushed
        C.moe_tiles(self.recv_counts, self.bn, self.r_offsets, self.tile_group, self.tile_tok0, self.tile_ntok,
                    self.meta)
        F = self.F
        C.wgemm(w_gate_up.view(self.per * 2 * F, H), self.recv_x, self.h, None, None, None, F, True, F, self.bn, 1,
                None, None, ws.status, self.tile_group, self.tile_tok0, self.tile_ntok, self.meta, self.max_tiles,
                2 * F, 0, [])
        C.wgemm(w_down.view(self.per * H, F), self.h, self.y_pairs, None, self.recv_w, self.recv_src, H, False, 0,
                self.bn, 1, None, None, ws.status, self.tile_group, self.tile_tok0, self.tile_ntok, self.meta,
                self.max_tiles, H, 0, self.y_peer)
        C.ep_sync(*peers, 48, True, self.seq, True, self.budget_ns, self.status)            # all results landed
        if out is None:
            out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
        C.moe_combine(self.y_pairs[:P], ids, 0, self.E, shared, shared_gate, residual, out, None, 0.0, 0.0, None)
        return out

    def check(self):
        v = int(self.status.item())
        if v:
            self._failed = f"expert-parallel exchange failed with device status {v}"
            raise EpError(self._failed)
