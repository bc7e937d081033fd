"""Symmetric-memory communicator: the host side of the fused reduction kernels (``csrc/comm.cu``).

Every rank allocates the same buffer through ``torch.distributed._symmetric_memory`` (CUDA VMM
allocations exchanged between the processes and mapped into every rank's address space), which gives
each rank the peer-mapped base pointer of every other rank's buffer and signal pad. The buffer holds
a small ring of "partial" slots: the o-proj / down-proj GEMM writes its rank-partial output straight
into the next slot (``next_partial``) and ``all_reduce_add_norm`` launches ONE kernel that signals the
peers, waits for them (bounded), sums all ranks' slots in rank order with NVLink peer loads, adds the
residual and applies the next RMSNorm. Sequence numbers live in device memory, so the calls can be
captured in a CUDA graph and replayed.

Slots rotate so that a rank never overwrites a slot a slower peer may still be reading: two different
slots for consecutive reductions, and ``end_step`` pads a step to an even number of reductions so the
rotation also holds across graph replays. Failure handling: a peer that does not arrive within the
deadline sets the status word (``check``); the communicator is then final (every later call raises),
like the reference's "first error is final" communicator (``src/tp_net/comm.rs:12-16``).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops.sm100 import ext


class CommError(RuntimeError):
    pass


class SymmComm:
    N_SLOTS = 2
    TWO_SHOT_ROWS = 512
    LL_ROWS = 64          # decode-sized reductions push flag-carrying lines instead of exchanging flags and loading
    AX_ROWS = 1024        # rows of one arg-max pair exchange (vocabulary-split head)

    def __init__(self, group, rank: int, world: int, device: torch.device, max_rows: int, hidden: int,
                 budget_ns: int = 5_000_000_000):
        from .dist import no_multicast_default
        no_multicast_default()
        import torch.distributed._symmetric_memory as symm_mem
        self.rank, self.world, self.device = rank, world, device
        self.max_rows, self.hidden = max_rows, hidden
        self.slot_bytes = max_rows * hidden * 2
        # regions after the partial slots: one for the two-shot reduce-scatter results, two that the all-gather
        # shards alternate between (see shard_view)
        self.rs_off = self.N_SLOTS * self.slot_bytes
        self.ag_off = (self.rs_off + self.slot_bytes, self.rs_off + 2 * self.slot_bytes)
        self._ag_half = 0
        self.ll_off = self.slot_bytes * (self.N_SLOTS + 3)
        self.ax_off = self.ll_off + 2 * world * self.LL_ROWS * hidden * 4
        nbytes = self.ax_off + 2 * world * self.AX_ROWS * 16
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.buf, group=group)
        self.buffer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.signal_ptrs = [int(p) for p in self.handle.signal_pad_ptrs]
        self.base = self.buf.data_ptr()
        assert self.base == self.buffer_ptrs[rank]
        # NVLink multicast address of the buffer (0 = not bound): with LB_MULTIMEM=1 the prompt-sized reduction loads
        # each element ONCE, already summed over the ranks inside the switch (multimem.ld_reduce), and stores the
        # result into every rank's region with one multicast store (multimem.st)
        import os
        self.mc_ptr = 0
        if os.environ.get("LB_MULTIMEM", "0") == "1":
            try:
                self.mc_ptr = int(self.handle.multicast_ptr or 0)
            except Exception:
                self.mc_ptr = 0
        self.seq = torch.zeros(1, dtype=torch.int32, device=device)
        self.done = torch.zeros(1, dtype=torch.int32, device=device)
        self.gemm_ctrs = torch.zeros(2, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.budget_ns = budget_ns
        self._next = 0
        self._calls_in_step = 0
        self._failed: Optional[str] = None
        self.buf.zero_()
        torch.cuda.synchronize(device)
        import torch.distributed as dist
        dist.barrier(group=group)

    # ------------------------------------------------------------------ slots
    def next_partial(self, rows: int, cols: int) -> Optional[torch.Tensor]:
        if rows > self.max_rows or cols != self.hidden:
            return None
        off = self._next * self.slot_bytes
        return self.buf[off:off + rows * cols * 2].view(torch.bfloat16).view(rows, cols)

    def owns(self, t: torch.Tensor) -> bool:
        p = t.data_ptr()
        return self.base <= p < self.base + self.slot_bytes * self.N_SLOTS and t.is_contiguous()

    def _advance(self):
        self._next = (self._next + 1) % self.N_SLOTS
        self._calls_in_step += 1

    # ------------------------------------------------------------------ collectives
    def all_reduce_add_norm(self, cur, res, w, eps, w_offset, quant: bool = False, combine=None):
        """cur must live in the current slot. Returns (normed, summed); with ``quant`` (decode-sized steps, a norm
        given) also the normalised rows NVFP4-encoded (``ops.sm100.Nv4Act``) out of the same launch. ``combine``
        (``ops.sm100.PendingCombine``, decode sizes): ``cur`` is the empty current slot and the launch first sums this
        rank's weighted expert rows per token into it."""
        if self._failed:
            raise CommError(self._failed)
        T, H = cur.shape
        if combine is not None and not (T <= self.LL_ROWS and H == self.hidden):
            combine.materialize(cur)
            combine = None
        off = cur.data_ptr() - self.base
        summed = torch.empty(T, H, dtype=torch.bfloat16, device=self.device)
        if T >= self.TWO_SHOT_ROWS and (self.world > 2 or self.mc_ptr):
            # two-shot: each rank reduces its block of rows (+ residual) into its own result region,
            # then every rank gathers all blocks; the norm runs on the gathered rows. With the multicast mapping
            # the reduction is one switch-side load per element and the result lands in every rank's region.
            per = (T + self.world - 1) // self.world
            row0 = min(T, self.rank * per)
            n_rows = max(0, min(T, row0 + per) - row0)
            out_off = self.rs_off      # rewritten only after the next call's flag round: every peer has left this one
            C = ext()
            C.reduce_scatter_fused(self.buffer_ptrs, self.signal_ptrs, self.rank, off, out_off, 0, self.seq, self.done,
                                   row0, n_rows, H, res, self.budget_ns, self.status, self.mc_ptr)
            C.all_gather_fused(self.buffer_ptrs, self.signal_ptrs, self.rank, out_off, 0, self.seq, self.done, T, H,
                               summed, self.budget_ns, self.status, bool(self.mc_ptr))
            self._advance()
            normed = None
            if w is not None:
                from ..ops import sm100
                normed, _ = sm100.rmsnorm(summed, w, eps, w_offset)
            if quant:
                from ..ops import sm100
                return normed, summed, sm100.nv4_quant_act(normed, key="ffn_in")
            return normed, summed
        normed = torch.empty_like(summed) if w is not None else None
        qc = qs = qg = None
        if quant:
            from ..ops import sm100
            C = ext()
            ws = sm100.Workspace.get(self.device)
            qc = ws.buf(("ar_q", "c"), (T, H // 2), torch.uint8)
            qs = ws.buf(("ar_q", "s"), (C.nv4_sf_bytes(T, H),), torch.uint8)
            qg = ws.buf(("ar_q", "g"), (max(T, 1),), torch.float32)
        from ..ops.sm100 import TUNE
        ll = self.LL_ROWS if (T <= self.LL_ROWS and H == self.hidden and TUNE.get("ar_ll", 1)) else 0
        if combine is not None and not ll:
            combine.materialize(cur)
            combine = None
        cm = combine
        ext().all_reduce_fused(self.buffer_ptrs, self.signal_ptrs, self.rank, off, 0, self.seq, self.done, T, H, res,
                               summed, w, eps, w_offset, normed, self.budget_ns, self.status, qc, qs, qg, self.ll_off, ll,
                               cm.y if cm else None, cm.ids if cm else None, cm.e_lo if cm else 0,
                               cm.e_hi if cm else 0, cm.shared if cm else None)
        self._advance()
        if quant:
            return normed, summed, sm100.Nv4Act(qc, qs, qg, 1, normed, summed)
        return normed, summed

    def fits_gemm_tail(self, rows: int, cols: int) -> bool:
        """One-shot sizes only: large steps keep the two-shot reduce-scatter + all-gather kernels."""
        return (rows <= self.max_rows and cols == self.hidden
                and not (rows >= self.TWO_SHOT_ROWS and (self.world > 2 or self.mc_ptr)))

    def linear_reduce_norm(self, x, w, res, norm_w, eps, w_offset):
        """(normed, summed) of sum_ranks(x @ w^T) + res in ONE launch: the GEMM writes this rank's partial tiles
        into the current slot and the same kernel's tail signals the peers, waits for them (bounded), sums all
        ranks' slots in rank order over NVLink peer loads, adds the residual and applies the norm."""
        if self._failed:
            raise CommError(self._failed)
        from ..ops import sm100
        T, N = x.shape[0], w.shape[0]
        slot = self.next_partial(T, N)
        off = slot.data_ptr() - self.base
        ws = sm100.Workspace.get(self.device)
        bn = sm100.pick_bn(T, False)
        n_tt, ft = (T + bn - 1) // bn, (N + 127) // 128
        sk = sm100._pick_split_k(n_tt, ft, x.shape[1])
        C = ext()
        if sk > 1 and (C.wgemm_workspace_floats(bn, False, n_tt, ft, sk) > ws.splitk.numel()
                       or n_tt * ft > ws.counters.numel()):
            sk = 1
        summed = torch.empty(T, N, dtype=torch.bfloat16, device=self.device)
        normed = torch.empty_like(summed) if norm_w is not None else None
        C.wgemm_allreduce(w, x, slot, bn, sk, ws.splitk if sk > 1 else None, ws.counters if sk > 1 else None,
                          ws.status, self.buffer_ptrs, self.signal_ptrs, self.rank, off, 0, self.seq, self.gemm_ctrs,
                          res, summed, norm_w, eps, w_offset, normed, self.budget_ns, self.status)
        self._advance()
        return normed, summed

    # ------------------------------------------------------------------ all-gather -> GEMM in one kernel
    def shard_rows(self, T: int):
        """(first row, row count, rows per rank) of this rank's block of a [T, hidden] activation."""
        per = (T + self.world - 1) // self.world
        row0 = min(T, self.rank * per)
        return row0, max(0, min(T, row0 + per) - row0), per

    def shard_view(self, T: int) -> torch.Tensor:
        """Where this rank writes its block of rows (inside its symmetric buffer) before ``all_gather_linear``.

        Ordering contract: write the block into ``shard_view(T)``, then call ``all_gather_linear(T, ...)``, once each,
        in that order on the compute stream. Consecutive calls alternate between two regions. The kernel's head only
        waits for the peers to ENTER call n, so a fast rank may leave call n while a slower peer still copies its
        rows; it then writes call n+1's block into the OTHER region, and can reach the first region again (call
        n+2) only after call n+1's flag round, which every peer raises after it has finished call n."""
        row0, n, _ = self.shard_rows(T)
        off = self.ag_off[self._ag_half] + row0 * self.hidden * 2
        return self.buf[off:off + n * self.hidden * 2].view(torch.bfloat16).view(n, self.hidden)

    def all_gather_linear(self, T: int, w: torch.Tensor, residual=None, out_dtype=torch.bfloat16):
        """out[T, N] = gather_ranks(x)[T, hidden] @ w[N, hidden]^T (+ residual) in ONE launch: the GEMM kernel's head
        exchanges flags with the peers, copies every rank's row block over NVLink peer loads into its local
        operand tensor, and then runs the tcgen05 main loop over it. Each rank must have written its block into
        ``shard_view(T)``. Returns (out, gathered activations)."""
        if self._failed:
            raise CommError(self._failed)
        if T > self.max_rows or w.shape[1] != self.hidden:
            raise CommError("all_gather_linear outside the communicator's shape")
        from ..ops import sm100
        C = ext()
        N = w.shape[0]
        ws = sm100.Workspace.get(self.device)
        x_full = ws.buf("ag_x", (self.max_rows, self.hidden), torch.bfloat16)[:T]
        out = torch.empty(T, N, dtype=out_dtype, device=self.device)
        bn = sm100.pick_bn(T, False)
        n_tt, ft = (T + bn - 1) // bn, (N + 127) // 128
        sk = sm100._pick_split_k(n_tt, ft, self.hidden)
        if sk > 1 and (C.wgemm_workspace_floats(bn, False, n_tt, ft, sk) > ws.splitk.numel()
                       or n_tt * ft > ws.counters.numel()):
            sk = 1
        _, _, per = self.shard_rows(T)
        C.wgemm_allgather(w, x_full, out, residual, bn, sk, ws.splitk if sk > 1 else None,
                          ws.counters if sk > 1 else None, ws.status, self.buffer_ptrs, self.signal_ptrs, self.rank,
                          self.ag_off[self._ag_half], 0, self.seq, self.gemm_ctrs, per, self.budget_ns, self.status)
        self._ag_half ^= 1
        return out, x_full

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        T, H = x.shape
        if not self.owns(x):
            slot = self.next_partial(T, H)
            if slot is None:
                raise CommError(f"all_reduce of {tuple(x.shape)} exceeds the symmetric buffer")
            slot.copy_(x)
            x = slot
        _, summed = self.all_reduce_add_norm(x, None, None, 0.0, 0.0)
        return summed

    def argmax_exchange(self, val: torch.Tensor, idx: torch.Tensor, vocab_offset: int, picks: torch.Tensor):
        """Greedy token per row from every rank's (best value, index inside its vocabulary slice): one launch that
        pushes the pairs to the peers and picks the global best (larger value, then lower token id) on every rank."""
        if self._failed:
            raise CommError(self._failed)
        if val.numel() > self.AX_ROWS:
            raise CommError("arg-max exchange of more rows than its area holds")
        ext().argmax_exchange(self.buffer_ptrs, self.signal_ptrs, self.rank, self.ax_off, self.AX_ROWS, self.seq,
                              self.done, val, idx, int(vocab_offset), picks, self.budget_ns, self.status)
        return picks

    def end_step(self):
        """Pads the step to an even number of reductions (slot rotation across graph replays)."""
        if self._calls_in_step % self.N_SLOTS:
            z = self.next_partial(1, self.hidden)
            z.zero_()
            self.all_reduce_add_norm(z, None, None, 0.0, 0.0)
        self._calls_in_step = 0

    def check(self):
        """Synchronises and raises if a bounded wait ran out; after that the communicator stays failed."""
        v = int(self.status.item())
        if v:
            self._failed = f"collective failed with device status {v} (a peer did not arrive in time)"
            raise CommError(self._failed)
