"""Pipeline parallelism: the layers are split over the ranks, the residual stream travels by point-to-point
send / recv (NCCL p2p on GPUs, gloo on CPU ranks), and a long prompt chunk is cut into micro-chunks so that
stage s works on micro-chunk c while stage s+1 works on c-1 (a wavefront without host round trips: the receive of
the next micro-chunk is posted before the current one is computed, sends are asynchronous).

Every rank runs the same scheduler in lock step (``parallel/spmd.py``) and builds the same ``StepBatch``; a rank
executes only its own layers on it and keeps KV / recurrent state only for those layers. The last stage computes
the final norm and the LM head and broadcasts the logit rows, so every rank samples the same tokens.

Reference counterparts: ``Executor`` stages with wavefront rounds (``src/model/core/exec.rs``), the dataflow
mailbox for long prompts (``src/model/core/exec/dataflow.rs``), ``--layer-split`` / ``--pipeline-micro``
(``docs/serving.md``). The chunk hand-off stays on the library's send / recv by design: it is bandwidth-trivial
(one [tokens, hidden] tensor per boundary) and overlaps with compute on the communication stream.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch


def split_layers(n_layer: int, world: int, layer_split: Optional[Sequence[int]] = None, last_extra: int = 0):
    """Stage boundaries. ``layer_split`` gives the layer counts per stage; otherwise the layers are spread evenly
    with the remainder on the first stages, and ``last_extra`` layers' worth of room is left on the last stage
    (it also runs the final norm and the LM head)."""
    if layer_split:
        counts = list(layer_split)
        if len(counts) != world or sum(counts) != n_layer or min(counts) < 0:
            raise ValueError(f"--layer-split {counts} does not cover {n_layer} layers on {world} stages")
    else:
        counts = [n_layer // world + (1 if r < n_layer % world else 0) for r in range(world)]
        move = min(last_extra, counts[-1]) if world > 1 else 0
        counts[-1] -= move
        for i in range(move):
            counts[i % (world - 1)] += 1
    bounds = [0]
    for c in counts:
        bounds.append(bounds[-1] + c)
    return bounds


class PipeStage:
    def __init__(self, rank: int, world: int, group, n_layer: int, layer_split: Optional[Sequence[int]] = None,
                 micro_tokens: int = 2048, last_extra: int = 0, decode_groups: int = 1):
        self.rank, self.world, self.group = rank, world, group
        self.bounds = split_layers(n_layer, world, layer_split, last_extra)
        self.lo, self.hi = self.bounds[rank], self.bounds[rank + 1]
        self.first, self.last = rank == 0, rank == world - 1
        self.micro_tokens = micro_tokens
        # decode steps: the running sequences travel the stages as this many groups, one behind the other, so
        # that stage s works on group g while stage s + 1 works on group g - 1 (``--pipeline-groups``; the
        # reference keeps decoding groups in flight the same way, ``src/engine/lm/pipe.rs:139``)
        self.decode_groups = max(1, decode_groups)
        self.stats = {"micro_chunks": 0, "decode_groups": 0, "sends": 0, "bytes": 0}

    def owns(self, il: int) -> bool:
        return self.lo <= il < self.hi

    # ------------------------------------------------------------------ micro-chunks
    def plan(self, b) -> List:
        """A step that is one sequence's prompt chunk longer than ``micro_tokens`` becomes several consecutive
        sub-steps over the same block table and state slot; any other step is one unit."""
        from ..models.decoder import StepBatch
        if b.rope_table is not None or b.deepstack is not None or b.slots_ring is not None:
            return [b]                # image tokens carry per-row inputs of their own: the step stays whole
        T = int(b.token_ids.shape[0]) if b.embeds is None else int(b.embeds.shape[0])
        if (self.decode_groups > 1 and b.max_q_len == 1 and b.embeds is None and T == b.n_seqs and T >= 2 * self.decode_groups
                and b.write_state and not b.capture_layers and b.replay is None):
            # a decode step: contiguous groups of sequences, each a complete step of its own
            per = (T + self.decode_groups - 1) // self.decode_groups
            out = []
            for a in range(0, T, per):
                e = min(T, a + per)
                out.append(StepBatch(
                    token_ids=b.token_ids[a:e], positions=b.positions[a:e],
                    cu_q=torch.arange(e - a + 1, dtype=torch.int32, device=b.cu_q.device), ctx_lens=b.ctx_lens[a:e],
                    block_table=b.block_table[a:e], slots=b.slots[a:e], state_slots=b.state_slots[a:e],
                    logit_rows=None, max_q_len=1, max_ctx=b.max_ctx, write_state=True, embeds=None,
                    cu_q_host=list(range(e - a + 1)), decode_splits=b.decode_splits))
            self.stats["decode_groups"] += len(out)
            return out
        if b.n_seqs != 1 or T <= self.micro_tokens or not b.write_state or b.capture_layers:
            return [b]
        out = []
        for a in range(0, T, self.micro_tokens):
            e = min(T, a + self.micro_tokens)
            out.append(StepBatch(
                token_ids=b.token_ids[a:e], positions=b.positions[a:e],
                cu_q=torch.tensor([0, e - a], dtype=torch.int32, device=b.cu_q.device),
                ctx_lens=b.ctx_lens - (T - e), block_table=b.block_table, slots=b.slots[a:e],
                state_slots=b.state_slots, logit_rows=None, max_q_len=e - a,
                max_ctx=(b.max_ctx - (T - e)) if b.max_ctx else 0, write_state=True,
                embeds=None if b.embeds is None else b.embeds[a:e], cu_q_host=[0, e - a],
                decode_splits=b.decode_splits))
        self.stats["micro_chunks"] += len(out)
        return out

    # ------------------------------------------------------------------ links
    def isend(self, t: torch.Tensor):
        import torch.distributed as dist
        self.stats["sends"] += 1
        self.stats["bytes"] += t.numel() * t.element_size()
        return dist.isend(t.contiguous(), dst=self.rank + 1, group=self.group)

    def irecv(self, rows: int, cols: int, dtype, device):
        import torch.distributed as dist
        buf = torch.empty(rows, cols, dtype=dtype, device=device)
        return buf, dist.irecv(buf, src=self.rank - 1, group=self.group)

    def broadcast_from_last(self, t: torch.Tensor):
        import torch.distributed as dist
        dist.broadcast(t, src=self.world - 1, group=self.group)
        return t
