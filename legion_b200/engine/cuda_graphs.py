"""CUDA-graph replay of decode steps.

A decode step's kernel sequence depends only on the number of rows: block tables, positions, lengths,
KV cells and state slots are tensors the kernels read. So one graph is captured per batch-size bucket
and replayed with new data: every step is ONE packed host-to-device copy of the step's integers from
pinned memory, one graph launch, and one small device-to-host copy of the picked tokens.

Reference counterpart: kept graphs per ``GroupShape`` and stage CUDA graphs with packed pinned inputs
(``src/model/core.rs:607-657``, ``src/ggml/stage_graph.rs:1-40``, ``src/ggml/pinned_io.rs``).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import ops
from ..kv import blocks as kv_blocks
from ..models.decoder import StepBatch

BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)


class _Entry:
    __slots__ = ("graph", "B", "W", "pack_h", "pack_d", "batch", "picks", "picks_h", "logits", "n_ints", "arange",
                 "bt_key", "pack_np", "all_picks", "all_picks_h", "logits_local")


class DecodeGraphs:
    def __init__(self, engine, want_logits: bool = False):
        self.eng = engine
        self.entries: Dict[int, _Entry] = {}
        self.want_logits = want_logits
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.replays = 0
        self.pad_slot = engine.cfg.max_seqs + (engine.cfg.prefix_cache_states if engine.saved is not None else 0)

    def bucket(self, n: int) -> Optional[int]:
        for b in BUCKETS:
            if n <= b:
                return b
        return None

    def release(self):
        """Destroys every captured graph and its private memory pool."""
        import gc
        if self.entries and torch.cuda.is_available():
            torch.cuda.synchronize(self.eng.device)
        self.entries.clear()
        gc.collect()

    def _layout(self, B: int, W: int):
        # int32 words: slots (int64 -> 2 words each) first so the int64 view is 8-byte aligned
        off = {}
        o = 0
        for name, n in (("slots", 2 * B), ("token_ids", B), ("positions", B), ("cu_q", B + 1), ("ctx_lens", B),
                        ("state_slots", B), ("block_table", B * W)):
            off[name] = (o, n)
            o += n
        return off, o

    def _lanes(self, B: int) -> int:
        """Concurrent lanes of a decode step: from 64 rows the batch runs as two independent halves on parallel
        branches of the graph. Each half stays within the 32-token tiles that the decode-sized kernels are tuned
        for (several CTAs per SM in the expert GEMMs, one dense-routing tile per expert), and the two chains fill
        each other's gaps: 16.1 against 18.0 ms per step at 64 users of the 80B-A3B shape. Below that it loses: at
        16 users two lanes of 8 took 8.7 ms against 6.8 ms, because every decode kernel occupies the whole machine
        while it waits on its own dependent hand-overs, so the lanes alternate instead of overlapping. One lane also
        for ranks that take part in collectives (their order must be the same on every rank) and for offloaded
        experts."""
        eng = self.eng
        pc = eng.model.pctx
        if B < 64 or B % 2 or getattr(pc, "world", 1) > 1 or eng.dp_world > 1 or eng.model.expert_cache:
            return 1
        return 2 if int(ops.sm100.TUNE.get("decode_lanes", 1)) >= 2 else 1

    def _capture(self, B: int) -> _Entry:
        eng = self.eng
        dev = eng.device
        W = eng.pool.blocks_for(eng.cfg.ctx_size)
        off, total = self._layout(B, W)
        e = _Entry()
        e.B, e.W, e.n_ints = B, W, total
        e.arange = torch.arange(B + 1, dtype=torch.int32)
        e.bt_key = [None] * B
        e.all_picks = e.all_picks_h = None
        e.pack_h = torch.zeros(total, dtype=torch.int32).pin_memory()
        e.pack_np = e.pack_h.numpy()          # the same pinned words, as the view the native packer writes
        e.pack_d = torch.zeros(total, dtype=torch.int32, device=dev)

        def view(name):
            o, n = off[name]
            return e.pack_d[o:o + n]

        Hkv = eng.model.n_kv_l
        G = max(1, eng.model.n_head_l // Hkv)
        splits = ops.sm100.decode_splits(B, Hkv, (G + 15) // 16, eng.cfg.ctx_size)
        e.batch = StepBatch(
            token_ids=view("token_ids"), positions=view("positions"), cu_q=view("cu_q"), ctx_lens=view("ctx_lens"),
            block_table=view("block_table").view(B, W), slots=view("slots").view(torch.int64),
            state_slots=view("state_slots"), logit_rows=None, max_q_len=1, max_ctx=eng.cfg.ctx_size,
            write_state=True, cu_q_host=list(range(B + 1)), decode_splits=splits)
        # neutral contents for warm-up and capture: every row is a padding row
        self._fill_padding(e, 0)
        e.pack_d.copy_(e.pack_h)
        e.picks = torch.zeros(B, dtype=torch.int32, device=dev)
        e.picks_h = torch.zeros(B, dtype=torch.int32).pin_memory()
        e.logits = None
        e.logits_local = None
        lanes = self._lanes(B)
        if lanes == 1:
            parts = [(e.batch, 0, B)]
        else:
            h = B // 2
            parts = []
            for lo, hi in ((0, h), (h, B)):
                n = hi - lo
                parts.append((StepBatch(
                    token_ids=view("token_ids")[lo:hi], positions=view("positions")[lo:hi],
                    cu_q=torch.arange(n + 1, dtype=torch.int32, device=dev), ctx_lens=view("ctx_lens")[lo:hi],
                    block_table=view("block_table").view(B, W)[lo:hi], slots=view("slots").view(torch.int64)[lo:hi],
                    state_slots=view("state_slots")[lo:hi], logit_rows=None, max_q_len=1, max_ctx=eng.cfg.ctx_size,
                    write_state=True, cu_q_host=list(range(n + 1)),
                    decode_splits=ops.sm100.decode_splits(n, Hkv, (G + 15) // 16, eng.cfg.ctx_size)), lo, hi))
            e.logits = torch.empty(B, eng.mcfg.vocab, dtype=torch.float32, device=dev)
        WS = ops.sm100.Workspace

        def run_lane(i):
            b, lo, hi = parts[i]
            WS.lane = i
            try:
                if eng.model.head_split is not None:
                    # vocabulary-split head: only (value, token id) pairs cross the ranks inside the graph; the
                    # logits stay per rank and are gathered after the replay for the rows that need them
                    out = eng.model.forward(b, eng.kv, eng.states, want_logits=False)
                    e.logits_local = eng.model.greedy_picks(out.hidden, e.picks[lo:hi])
                    return out
                out = eng.model.forward(b, eng.kv, eng.states)
                ops.sm100.argmax(out.logits, out=e.picks[lo:hi])
                if lanes > 1:
                    e.logits[lo:hi].copy_(out.logits)
                return out
            finally:
                WS.lane = 0

        s = torch.cuda.Stream(device=dev)
        s.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(s):
            for _ in range(2):   # warm-up outside capture: allocates workspaces, tensor maps, attributes
                for i in range(lanes):
                    run_lane(i)
        torch.cuda.current_stream(dev).wait_stream(s)
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        side = [torch.cuda.Stream(device=dev) for _ in range(lanes - 1)]
        with torch.cuda.graph(g):
            main = torch.cuda.current_stream(dev)
            if lanes > 1:
                fork = torch.cuda.Event()
                fork.record(main)
            out = run_lane(0)
            for i, st in enumerate(side):
                st.wait_event(fork)
                with torch.cuda.stream(st):
                    run_lane(i + 1)
                    join = torch.cuda.Event()
                    join.record(st)
                main.wait_event(join)
            if lanes == 1 and eng.model.head_split is None:
                e.logits = out.logits
        e.graph = g
        self.entries[B] = e
        return e

    def _fill_padding(self, e: _Entry, n_real: int):
        off, _ = self._layout(e.B, e.W)
        h = e.pack_h
        o, n = off["slots"]
        h[o + 2 * n_real:o + n].view(torch.int64).fill_(-1)
        for name, val in (("token_ids", 0), ("positions", 0), ("ctx_lens", 1), ("state_slots", self.pad_slot)):
            o, n = off[name]
            h[o + n_real:o + n] = val
        o, n = off["block_table"]
        h[o + n_real * e.W:o + n] = 0

    def run(self, rows, B: Optional[int] = None, gather=None) -> Tuple[Optional[List[int]], Optional[torch.Tensor]]:
        """rows: [(seq, position, 1)]. Returns (picked token per row, logits [n, V]) or (None, None) when the
        batch does not fit a bucket. ``B`` forces the bucket (data-parallel attention: every rank replays the
        bucket of the fullest rank, possibly with no row of its own) and ``gather=(group, world)`` makes the
        result the picks of ALL ranks, ``world * B`` values in rank order."""
        n = len(rows)
        B = B or self.bucket(n)
        if B is None:
            return None, None
        e = self.entries.get(B) or self._capture(B)
        eng = self.eng
        pool = eng.pool
        native = kv_blocks.NATIVE
        if native is not None:
            # the whole record is written by one call of the native host runtime
            native.pack_decode(e.pack_np, B, e.W, pool.block_size, self.pad_slot,
                               [s.tokens[-1] for s, _, _ in rows], [p0 for _, p0, _ in rows],
                               [s.slot for s, _, _ in rows], [s.table.blocks for s, _, _ in rows])
            if any(s.media is not None and s.media.rope_delta for s, _, _ in rows):
                # sequences with images: rotary positions run behind the token index by a constant
                off, _ = self._layout(B, e.W)
                ps = e.pack_h[off["positions"][0]:off["positions"][0] + B]
                for i, (s, p0, _) in enumerate(rows):
                    if s.media is not None:
                        ps[i] = s.rope_pos(p0)
            return self._replay(e, rows, n, B, gather)
        off, _ = self._layout(B, e.W)
        h = e.pack_h
        sl = h[off["slots"][0]:off["slots"][0] + 2 * B].view(torch.int64)
        tk = h[off["token_ids"][0]:off["token_ids"][0] + B]
        ps = h[off["positions"][0]:off["positions"][0] + B]
        cl = h[off["ctx_lens"][0]:off["ctx_lens"][0] + B]
        ss = h[off["state_slots"][0]:off["state_slots"][0] + B]
        bt = h[off["block_table"][0]:off["block_table"][0] + B * e.W].view(B, e.W)
        cu = h[off["cu_q"][0]:off["cu_q"][0] + B + 1]
        cu.copy_(e.arange)
        bs = pool.block_size
        p0s = [p0 for _, p0, _ in rows]
        sl[:n] = torch.tensor([s.table.blocks[p0 // bs] * bs + p0 % bs for s, p0, _ in rows], dtype=torch.int64)
        tk[:n] = torch.tensor([s.tokens[-1] for s, _, _ in rows], dtype=torch.int32)
        pt = torch.tensor(p0s, dtype=torch.int32)
        ps[:n] = torch.tensor([s.rope_pos(p0) for s, p0, _ in rows], dtype=torch.int32)
        cl[:n] = pt + 1
        ss[:n] = torch.tensor([s.slot for s, _, _ in rows], dtype=torch.int32)
        for i, (s, p0, _) in enumerate(rows):
            # a sequence's block table only changes when it crosses into a new block
            key = (id(s), len(s.table.blocks), s.table.blocks[0], s.table.blocks[-1])
            if e.bt_key[i] != key:
                nb = len(s.table.blocks)
                bt[i, :nb] = torch.tensor(s.table.blocks, dtype=torch.int32)
                e.bt_key[i] = key
        for i in range(n, B):
            e.bt_key[i] = None
        self._fill_padding(e, n)
        return self._replay(e, rows, n, B, gather)

    def _replay(self, e: _Entry, rows, n: int, B: int, gather=None):
        eng = self.eng
        e.pack_d.copy_(e.pack_h, non_blocking=True)
        e.graph.replay()
        if gather is not None:
            import torch.distributed as dist
            group, world = gather
            if e.all_picks is None:
                e.all_picks = torch.zeros(world * B, dtype=torch.int32, device=eng.device)
                e.all_picks_h = torch.zeros(world * B, dtype=torch.int32).pin_memory()
            dist.all_gather_into_tensor(e.all_picks, e.picks, group=group)
            e.all_picks_h.copy_(e.all_picks, non_blocking=True)
            torch.cuda.current_stream(eng.device).synchronize()
            self.h2d_bytes += e.n_ints * 4
            self.d2h_bytes += world * B * 4
            self.replays += 1
            return e.all_picks_h.tolist(), None
        e.picks_h.copy_(e.picks, non_blocking=True)
        torch.cuda.current_stream(eng.device).synchronize()
        self.h2d_bytes += e.n_ints * 4
        self.d2h_bytes += B * 4
        self.replays += 1
        need_logits = any(not (s.req.sampling.greedy and s.req.sampling.plain and s.constraint is None)
                          for s, _, _ in rows)
        if need_logits and e.logits is None and e.logits_local is not None:
            return e.picks_h[:n].tolist(), eng.model.gather_logits(e.logits_local)[:n]
        return e.picks_h[:n].tolist(), (e.logits[:n] if need_logits else None)
