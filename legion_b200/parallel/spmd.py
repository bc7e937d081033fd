"""Serving with several ranks: rank 0 owns the HTTP server; every rank runs the SAME scheduler on the same
stream of requests, so all ranks plan identical steps and meet in the collectives without a per-step
descriptor exchange. Rank 0 publishes each admitted request (and each cancellation) on a CPU side channel
(a gloo group); followers replay them into their own engine at the same step boundary.

The reference's rank 0 likewise serves HTTP and leads, sending step descriptors to the other ranks over its
control connections (``src/tp_net.rs:5-6``, ``src/model/core/exec/tp_lead.rs:455``). A rank that stops
answering ends the group's next collective by timeout; the communicator error is final.
"""
from __future__ import annotations

import datetime
import pickle
import threading
from typing import List, Optional

import torch


class StepChannel:
    """Broadcast of per-step control messages from rank 0 over gloo (CPU tensors)."""

    def __init__(self, rank: int, world: int, timeout_s: float = 300.0):
        import torch.distributed as dist
        self.rank, self.world = rank, world
        self.group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))

    def exchange(self, msgs: Optional[list]) -> list:
        """Rank 0 passes its messages; every rank returns rank 0's list."""
        import torch.distributed as dist
        box = [msgs if self.rank == 0 else None]
        dist.broadcast_object_list(box, src=0, group=self.group)
        return box[0] or []


def attach(engine, rank: int, world: int, timeout_s: float = 600.0) -> StepChannel:
    """Puts the engine into lock-step mode (call on every rank before the engine thread starts)."""
    ch = StepChannel(rank, world, timeout_s)
    engine.channel = ch
    return ch


def follower_wait(engine) -> int:
    """Ranks > 0 have no HTTP server: they run the engine thread and wait for rank 0's shutdown message."""
    engine.start()
    while engine._thread is not None and engine._thread.is_alive():
        engine._thread.join(timeout=1.0)
    return 0
