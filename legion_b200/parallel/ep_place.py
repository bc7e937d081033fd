"""Co-activation aware expert placement for expert parallelism (``legion ep-place``).

Input: a route record, JSON lines ``{"layer": l, "experts": [e0, e1, ...]}`` (one line per routed token, written
with ``--moe-route-record``). Experts that fire together for the same token are cheapest when they sit on
different ranks (their work runs in parallel), and every rank should carry the same share of the load. The
placement is greedy: experts in order of decreasing load go to the rank with the lowest sum of load and
co-activation with what that rank already holds, under an equal-count cap
(``src/tp_net/ep_place.rs`` in the reference).
"""
from __future__ import annotations

import json
from collections import defaultdict
from typing import Dict, List


def place(load: Dict[int, float], co: Dict[tuple, float], n_expert: int, ranks: int) -> List[int]:
    cap = (n_expert + ranks - 1) // ranks
    owner = [-1] * n_expert
    held: List[List[int]] = [[] for _ in range(ranks)]
    rank_load = [0.0] * ranks
    for e in sorted(range(n_expert), key=lambda x: -load.get(x, 0.0)):
        best, best_cost = 0, None
        for r in range(ranks):
            if len(held[r]) >= cap:
                continue
            cost = rank_load[r] + sum(co.get((min(e, o), max(e, o)), 0.0) for o in held[r])
            if best_cost is None or cost < best_cost:
                best, best_cost = r, cost
        owner[e] = best
        held[best].append(e)
        rank_load[best] += load.get(e, 0.0)
    return owner


def place_from_record(path: str, ranks: int) -> dict:
    load: Dict[int, Dict[int, float]] = defaultdict(lambda: defaultdict(float))
    co: Dict[int, Dict[tuple, float]] = defaultdict(lambda: defaultdict(float))
    n_expert = 0
    for line in open(path):
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        l, ex = int(rec["layer"]), [int(e) for e in rec["experts"]]
        n_expert = max(n_expert, max(ex) + 1)
        for i, a in enumerate(ex):
            load[l][a] += 1.0
            for b in ex[i + 1:]:
                co[l][(min(a, b), max(a, b))] += 1.0
    n_expert = ((n_expert + ranks - 1) // ranks) * ranks
    out = {"ranks": ranks, "n_expert": n_expert, "layers": {}}
    for l in sorted(load):
        owner = place(load[l], co[l], n_expert, ranks)
        per_rank = [sum(load[l].get(e, 0.0) for e in range(n_expert) if owner[e] == r) for r in range(ranks)]
        out["layers"][str(l)] = {"owner": owner, "rank_load": per_rank}
    return out
