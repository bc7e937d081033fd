"""Memory plan: what a rank's HBM holds and how large the KV pool can be beside it.

At start-up the engine knows the bytes already resident (weights), the bytes of one KV block over all layers, the
bytes of one recurrent-state slot, and what the device reports as free. ``fit`` turns that into the number of KV
blocks (``--kv-cache-tokens auto``), the largest context that fits when the asked one does not, and the lines of
the plan that the engine logs. Reference counterparts: ``src/engine/lm/plan.rs`` (memory plan log), ``fit.rs`` /
``kv_fit.rs`` (largest context whose cache fits beside the measured compute buffers), ``vram.rs``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List

GIB = float(1 << 30)


@dataclass
class MemoryPlan:
    total_bytes: int
    free_bytes: int                 # free on the device before the pools are allocated
    weights_bytes: int
    workspace_bytes: int            # kept back for activations, kernel workspaces and CUDA-graph pools
    state_bytes: int                # recurrent-state slots (running sequences + saved snapshots)
    bytes_per_block: int
    block_size: int
    n_blocks: int
    asked_tokens: int               # max_seqs * ctx_size (or the explicit --kv-cache-tokens)
    fits: bool                      # the asked number of tokens fits
    max_ctx_fit: int                # largest context per sequence that fits for max_seqs sequences
    notes: List[str] = field(default_factory=list)

    @property
    def kv_bytes(self) -> int:
        return self.n_blocks * self.bytes_per_block

    @property
    def kv_tokens(self) -> int:
        return self.n_blocks * self.block_size

    def lines(self) -> List[str]:
        out = [f"memory plan: device {self.total_bytes / GIB:.1f} GiB, free {self.free_bytes / GIB:.1f} GiB",
               f"  weights      {self.weights_bytes / GIB:8.2f} GiB (resident)",
               f"  KV pool      {self.kv_bytes / GIB:8.2f} GiB = {self.n_blocks} blocks x {self.block_size} tokens "
               f"({self.bytes_per_block / 1024:.0f} KiB per block over all layers) = {self.kv_tokens} tokens",
               f"  state slots  {self.state_bytes / GIB:8.2f} GiB",
               f"  kept back    {self.workspace_bytes / GIB:8.2f} GiB (activations, workspaces, graph pools)"]
        if not self.fits:
            out.append(f"  asked for {self.asked_tokens} tokens: does not fit; largest context for the configured number "
                       f"of sequences is {self.max_ctx_fit}")
        return out + [f"  {n}" for n in self.notes]


def workspace_reserve(hidden: int, vocab: int, max_batch_tokens: int, max_seqs: int, n_expert: int, top_k: int,
                      expert_ff: int) -> int:
    """Bytes a step needs beside weights and pools: activations of the widest layer for a full batch, the logits of
    every sequence, the expert-sorted copies of a prompt-sized MoE step, split-K and attention workspaces, and the
    private pools of the captured decode graphs (one per batch bucket)."""
    T = max_batch_tokens
    act = T * hidden * 2 * 12                                  # residual, normed, projections, attention output ...
    moe = T * max(1, top_k) * (hidden + expert_ff) * 2 * 2 if n_expert else 0
    logits = max_seqs * vocab * 4 * 3
    fixed = (64 + 32 + 256) << 20                              # split-K, attention partials, graph pools
    return int(act + moe + logits + fixed)


def fit(total_bytes: int, free_bytes: int, weights_bytes: int, bytes_per_block: int, block_size: int,
        state_bytes: int, workspace_bytes: int, max_seqs: int, ctx_size: int, asked_tokens: int = 0,
        utilisation: float = 0.92) -> MemoryPlan:
    """``asked_tokens`` = 0: take what fits (at most max_seqs * ctx_size tokens are useful); otherwise check that the
    asked pool fits and size it exactly. ``utilisation``: share of the device's total memory this process may use."""
    budget = int(min(free_bytes, total_bytes * utilisation - (total_bytes - free_bytes))) - state_bytes - workspace_bytes
    can = max(0, budget // max(1, bytes_per_block))
    useful = (max_seqs * ctx_size + block_size - 1) // block_size
    want = (asked_tokens + block_size - 1) // block_size if asked_tokens > 0 else useful
    n_blocks = min(can, want)
    fits = can >= want
    per_seq_blocks = can // max(1, max_seqs)
    notes = []
    if asked_tokens <= 0 and can > useful:
        notes.append(f"{(can - useful) * bytes_per_block / GIB:.1f} GiB left unused: every sequence already has its whole context")
    return MemoryPlan(total_bytes, free_bytes, weights_bytes, workspace_bytes, state_bytes, bytes_per_block, block_size,
                      max(4, n_blocks) if fits or asked_tokens <= 0 else n_blocks, want * block_size, fits,
                      per_seq_blocks * block_size, notes)
