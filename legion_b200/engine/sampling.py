"""Host-side sampler: penalties -> logit bias -> temperature -> min-p -> top-k -> top-p -> one draw.

Used for rows that need logit edits, log-probabilities or exact rejection sampling; plain rows are
picked on the device (``ops.argmax`` / the sampling kernel). Order and semantics follow the reference
sampler (``src/engine/sampling.rs:1-12,118-162``): presence / frequency penalties count generated tokens
only, the repetition penalty divides positive and multiplies negative logits of every seen token,
temperature 0 means arg-max after penalties, draws come from a seeded SplitMix64 stream.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .types import SamplingParams

_MASK = (1 << 64) - 1


class SplitMix64:
    def __init__(self, seed: int):
        self.state = seed & _MASK

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
        return z ^ (z >> 31)

    def uniform(self) -> float:
        return (self.next_u64() >> 11) * (1.0 / (1 << 53))


class Sampler:
    """Per-sequence sampling state (RNG stream and token counts)."""

    def __init__(self, params: SamplingParams, prompt_tokens: Sequence[int], fallback_seed: int = 0):
        self.p = params
        self.rng = SplitMix64(params.seed if params.seed is not None else fallback_seed)
        self.gen_counts: Dict[int, int] = {}
        self.seen = set(prompt_tokens) if params.repetition_penalty != 1.0 else set()

    def accept(self, token: int):
        self.gen_counts[token] = self.gen_counts.get(token, 0) + 1
        if self.p.repetition_penalty != 1.0:
            self.seen.add(token)

    def adjusted(self, logits: torch.Tensor, mask: Optional[torch.Tensor] = None, eos_ids: Sequence[int] = (),
                 n_generated: int = 0) -> torch.Tensor:
        """Logits after penalties, bias, grammar mask and the min_tokens rule (float32, on the CPU)."""
        p = self.p
        lg = logits.detach().float().cpu().clone()
        if self.gen_counts and (p.presence_penalty or p.frequency_penalty):
            idx = torch.tensor(list(self.gen_counts.keys()), dtype=torch.long)
            cnt = torch.tensor(list(self.gen_counts.values()), dtype=torch.float32)
            lg[idx] -= p.presence_penalty + p.frequency_penalty * cnt
        if p.repetition_penalty != 1.0 and self.seen:
            idx = torch.tensor(sorted(self.seen), dtype=torch.long)
            v = lg[idx]
            lg[idx] = torch.where(v > 0, v / p.repetition_penalty, v * p.repetition_penalty)
        for tid, b in p.logit_bias.items():
            if 0 <= tid < lg.numel():
                lg[tid] += b
        if n_generated < p.min_tokens:
            for e in eos_ids:
                lg[e] = float("-inf")
        if mask is not None:
            lg = torch.where(mask, lg, torch.full_like(lg, float("-inf")))
        return lg

    def distribution(self, lg: torch.Tensor) -> torch.Tensor:
        """Final sampling distribution (sums to 1) for adjusted logits; a point mass when greedy."""
        p = self.p
        if p.greedy:
            d = torch.zeros_like(lg)
            d[int(torch.argmax(lg))] = 1.0
            return d
        pr = torch.softmax(lg / p.temperature, dim=-1)
        if p.min_p > 0:
            pr = torch.where(pr >= p.min_p * pr.max(), pr, torch.zeros_like(pr))
        if 0 < p.top_k < pr.numel():
            kth = torch.topk(pr, p.top_k).values[-1]
            pr = torch.where(pr >= kth, pr, torch.zeros_like(pr))
        if p.top_p < 1.0:
            sp, si = torch.sort(pr, descending=True, stable=True)
            tot = sp.sum()
            before = torch.cumsum(sp, 0) - sp
            keep = before < p.top_p * tot
            m = torch.zeros_like(pr, dtype=torch.bool)
            m[si[keep]] = True
            pr = torch.where(m, pr, torch.zeros_like(pr))
        return pr / pr.sum()

    def draw(self, dist: torch.Tensor) -> int:
        u = self.rng.uniform()
        c = torch.cumsum(dist.double(), 0)
        i = int(torch.searchsorted(c, torch.tensor(u * float(c[-1]), dtype=torch.float64), right=True))
        i = min(i, dist.numel() - 1)
        while dist[i] == 0 and i > 0:   # guard against a tie on a zero-probability boundary
            i -= 1
        return i

    def sample(self, logits: torch.Tensor, mask=None, eos_ids=(), n_generated=0) -> Tuple[int, torch.Tensor]:
        lg = self.adjusted(logits, mask, eos_ids, n_generated)
        if self.p.greedy:
            return int(torch.argmax(lg)), lg
        return self.draw(self.distribution(lg)), lg


def top_logprobs(lg: torch.Tensor, chosen: int, n: int) -> Tuple[float, List[Tuple[int, float]]]:
    lp = torch.log_softmax(lg.float(), dim=-1)
    top: List[Tuple[int, float]] = []
    if n > 0:
        v, i = torch.topk(lp, min(n, lp.numel()))
        top = [(int(a), float(b)) for a, b in zip(i.tolist(), v.tolist())]
    return float(lp[chosen]), top


def resolve_sampling_defaults(request: dict, operator: dict, model_file: dict, arch: dict) -> dict:
    """Precedence request > operator flags > model file > architecture > OpenAI defaults
    (``docs/serving.md:103-112`` of the reference)."""
    base = {"temperature": 1.0, "top_p": 1.0, "top_k": 0, "min_p": 0.0}
    for src in (arch, model_file, operator, request):
        for k, v in (src or {}).items():
            if v is not None:
                base[k] = v
    return base
