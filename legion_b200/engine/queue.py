"""Waiting queue of the scheduler: FCFS or priority order, optional fair sharing between keys
(API keys / users), and re-queueing of preempted requests ahead of new arrivals.

Reference: ``src/engine/queue.rs:34,183,250,278`` (WaitQueue, fair-share pop, requeue).
"""
from __future__ import annotations

import itertools
from collections import defaultdict, deque
from typing import Any, Deque, Dict, List, Optional


class WaitQueue:
    def __init__(self, policy: str = "fcfs", fair_share: bool = False, max_waiting: int = 1024):
        assert policy in ("fcfs", "priority")
        self.policy, self.fair_share, self.max_waiting = policy, fair_share, max_waiting
        self._items: List[tuple] = []      # (priority, seq_no, key, item)
        self._counter = itertools.count()
        self._served: Dict[Optional[str], int] = defaultdict(int)   # tokens served per key (fair share)

    def __len__(self):
        return len(self._items)

    def full(self) -> bool:
        return len(self._items) >= self.max_waiting

    def push(self, item: Any, priority: int = 0, key: Optional[str] = None):
        self._items.append((priority, next(self._counter), key, item))

    def requeue(self, item: Any, priority: int = 0, key: Optional[str] = None):
        """A preempted request goes back in front of everything of its priority."""
        self._items.append((priority, -next(self._counter), key, item))

    def _order(self, e):
        prio, no, key, _ = e
        # higher priority first; then (fair share) the key that has been served least; then arrival
        served = self._served[key] if self.fair_share else 0
        if self.policy == "priority":
            return (-prio, served, no)
        return (served, no)

    def peek(self):
        if not self._items:
            return None
        return min(self._items, key=self._order)[3]

    def pop(self):
        if not self._items:
            return None
        e = min(self._items, key=self._order)
        self._items.remove(e)
        return e[3]

    def remove(self, pred) -> List[Any]:
        out = [e[3] for e in self._items if pred(e[3])]
        self._items = [e for e in self._items if not pred(e[3])]
        return out

    def charge(self, key: Optional[str], tokens: int):
        self._served[key] += tokens

    def by_priority(self) -> Dict[int, int]:
        d: Dict[int, int] = defaultdict(int)
        for prio, *_ in self._items:
            d[prio] += 1
        return dict(d)

    def n_keys(self) -> int:
        return len({e[2] for e in self._items})

    def items(self) -> List[Any]:
        return [e[3] for e in sorted(self._items, key=self._order)]
