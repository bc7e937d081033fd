"""Draft depth from what was measured: per-sequence acceptance along a chain, and step costs.

``AdaptiveState`` (one per sequence; the reference's ``src/spec/adaptive.rs``): decayed counts of accepted drafts and
of draft positions tried give the probability ``rate`` that a draft is accepted given the drafts before it were; the
deepest draft whose LAST token still has at least ``p_floor`` acceptance probability (``rate ** k >= p_floor``) is the
sequence's cap. ``gains[k]`` keeps, decayed, what a step with a cap of k drafts would have gained: drafts do not
depend on the cap, so a verify step tells the gain of every smaller cap, and of larger ones too when the chain ended
before its cap; only a chain that reached its cap leaves larger caps to the geometric tail at ``rate``.

``DepthModel`` (one per engine; ``src/spec/depth.rs``): a step's verify cost ``V(rows)`` and the drafter's cost
``D(batch)`` per draft step are exponential averages (weight 0.2) of measured times, bucketed by powers of two; the
depth for a step maximises ``sum_s gain_s(k) / (V(b (1 + k)) + D(b) k)`` over k; a neighbouring depth is probed every
16 drafting steps so its cost stays known; the choice changes only when it is better by 2 % (hysteresis); unknown
costs fall back to a row-cost model."""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional

DECAY = 0.9            # per verify step, the weight the chain estimates keep of what they knew before
PRIOR_RATE = 0.6       # per-position acceptance of a sequence nothing is known about
MAX_GAIN_DEPTH = 16
EWMA = 0.2
PROBE_EVERY = 16
HYSTERESIS = 1.02


def chain_gain(a: float, k: int) -> float:
    """1 + a + a^2 + ... + a^k: tokens a chain of k drafts gains at per-position acceptance a (bonus included)."""
    if a >= 1.0:
        return float(k + 1)
    return (1.0 - a ** (k + 1)) / (1.0 - a)


class AdaptiveState:
    __slots__ = ("acc", "tried", "gains", "weight", "idle")

    def __init__(self):
        self.acc = PRIOR_RATE          # decayed accepted drafts ...
        self.tried = 1.0               # ... over decayed positions tried (one prior observation)
        self.gains = [0.0] * (MAX_GAIN_DEPTH + 1)
        self.weight = 0.0              # decayed number of steps behind ``gains``
        self.idle = 0                  # consecutive steps in which the cap was 0

    @property
    def rate(self) -> float:
        return min(0.999, max(0.0, self.acc / self.tried)) if self.tried > 0 else PRIOR_RATE

    def update(self, drafted: int, accepted: int, cap: int) -> None:
        """After verifying ``drafted`` drafts made under cap ``cap``, the first ``accepted`` of which were accepted."""
        if drafted <= 0:
            return
        ended_early = accepted < drafted or drafted < cap       # a rejection, or a draft the head declined to make
        self.acc = self.acc * DECAY + accepted
        self.tried = self.tried * DECAY + accepted + (1 if ended_early else 0)
        r = self.rate
        self.weight = self.weight * DECAY + 1.0
        for k in range(MAX_GAIN_DEPTH + 1):
            if k <= drafted or ended_early:
                g = 1.0 + min(accepted, k)
            else:                                               # reached its cap: larger caps get the geometric tail
                g = 1.0 + accepted + sum(r ** i for i in range(1, k - drafted + 1))
            self.gains[k] = self.gains[k] * DECAY + g
        self.idle = 0

    def gain(self, k: int) -> float:
        """Expected tokens of a step with a cap of k drafts (bonus included)."""
        k = min(k, MAX_GAIN_DEPTH)
        if self.weight < 0.5:
            return chain_gain(self.rate, k)
        return self.gains[k] / self.weight

    def cap(self, p_floor: float, max_k: int) -> int:
        """Deepest draft whose last token keeps at least ``p_floor`` acceptance probability."""
        r, k, p = self.rate, 0, 1.0
        while k < max_k and p * r >= p_floor:
            p *= r
            k += 1
        return k

    def note_idle(self) -> bool:
        """A step without drafts for this sequence; every eighth one asks for a single probing draft so that a
        sequence whose acceptance recovered is noticed."""
        self.idle += 1
        return self.idle % 8 == 0


def _bucket(n: int) -> int:
    b = 1
    while b < n:
        b <<= 1
    return b


class DepthModel:
    def __init__(self, max_k: int, row_cost: float = 0.02):
        self.max_k = max_k
        self.row_cost = row_cost                  # fallback: relative cost of one more verify row next to a decode step
        self.verify_ms: Dict[int, float] = {}     # rows bucket -> ms
        self.draft_ms: Dict[int, float] = {}      # batch bucket -> ms per draft step
        self.steps = 0
        self.current = max_k
        self.last_probe: Optional[int] = None

    # ---- measurements
    def observe_verify(self, rows: int, ms: float) -> None:
        b = _bucket(max(1, rows))
        old = self.verify_ms.get(b)
        self.verify_ms[b] = ms if old is None else (1 - EWMA) * old + EWMA * ms

    def observe_draft(self, batch: int, k: int, ms: float) -> None:
        if k <= 0:
            return
        b = _bucket(max(1, batch))
        per = ms / k
        old = self.draft_ms.get(b)
        self.draft_ms[b] = per if old is None else (1 - EWMA) * old + EWMA * per

    def _verify_cost(self, rows: int) -> Optional[float]:
        b = _bucket(max(1, rows))
        if b in self.verify_ms:
            return self.verify_ms[b]
        known = sorted(self.verify_ms)
        if not known:
            return None
        lo = max((x for x in known if x < b), default=None)
        hi = min((x for x in known if x > b), default=None)
        if lo is not None and hi is not None:       # between two measured buckets: interpolate on the row count
            t = (b - lo) / (hi - lo)
            return self.verify_ms[lo] * (1 - t) + self.verify_ms[hi] * t
        base = self.verify_ms[lo if lo is not None else hi]
        ref = lo if lo is not None else hi
        return base * (1.0 + self.row_cost * (b - ref))

    # ---- choice
    def choose(self, states: Iterable[AdaptiveState], batch: int) -> int:
        """Depth for a step over ``batch`` drafting sequences with the given acceptance states."""
        states = list(states)
        if not states or self.max_k <= 0:
            return 0
        self.steps += 1
        base = self._verify_cost(batch)
        d_per = self.draft_ms.get(_bucket(batch), 0.0)

        def score(k: int) -> float:
            tokens = sum(s.gain(k) for s in states)
            v = self._verify_cost(batch * (1 + k))
            if v is None or base is None:
                cost = 1.0 + k * batch * self.row_cost
            else:
                cost = (v + d_per * k) / max(base, 1e-6)
            return tokens / max(cost, 1e-6)

        best = max(range(0, self.max_k + 1), key=score)
        if best != self.current and score(best) < HYSTERESIS * score(self.current):
            best = self.current
        self.current = best
        if self.steps % PROBE_EVERY == 0:
            # keep the neighbouring depths' costs known: alternate one deeper, one shallower
            up = self.last_probe != best + 1 and best < self.max_k
            probe = best + 1 if up else max(0 if best > 1 else 1, best - 1)
            self.last_probe = probe
            return min(self.max_k, probe)
        return best
