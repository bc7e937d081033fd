"""Data-parallel replicas: N whole engines (own scheduler, KV cache and prefix cache) behind one ``Engine``.

Routing (``src/engine/replicas.rs:1-30,123,192`` in the reference): a prompt of at least 256 tokens goes to the
replica whose prefix cache already holds at least half of it (prefix affinity); otherwise to the replica with
the fewest requests in flight, ties to the one with the most free KV blocks.
"""
from __future__ import annotations

from typing import List

from .types import Engine, EngineStats, GenerateRequest, TokenStream

AFFINITY_MIN_TOKENS = 256


class ReplicaEngine(Engine):
    def __init__(self, engines: List[Engine]):
        assert engines
        self.engines = engines

    def models(self):
        return self.engines[0].models()

    def check_response_format(self, fmt):
        self.engines[0].check_response_format(fmt)

    def count_tokens(self, req):
        return self.engines[0].count_tokens(req)

    def _load(self, e: Engine):
        st = e.stats()
        return (st.running + st.waiting, -(st.kv_blocks_total - st.kv_blocks_used))

    def pick(self, req: GenerateRequest) -> int:
        tokens = None
        e0 = self.engines[0]
        if hasattr(e0, "tokenize_request"):
            try:
                tokens = e0.tokenize_request(req)
            except Exception:
                tokens = None
        if tokens is not None and len(tokens) >= AFFINITY_MIN_TOKENS:
            best, best_n = -1, 0
            for i, e in enumerate(self.engines):
                radix = getattr(e, "radix", None)
                if radix is None:
                    continue
                _, n, _ = radix.match_prefix(tokens, lock=False)
                if n > best_n:
                    best, best_n = i, n
            if best >= 0 and best_n * 2 >= len(tokens):
                return best
        return min(range(len(self.engines)), key=lambda i: self._load(self.engines[i]))

    def generate(self, req: GenerateRequest) -> TokenStream:
        return self.engines[self.pick(req)].generate(req)

    def stats(self) -> EngineStats:
        agg = EngineStats()
        for s in self.replica_stats():
            for f in ("running", "waiting", "kv_blocks_used", "kv_blocks_total", "kv_preemptions",
                      "prefix_cache_hit_tokens", "prompt_tokens", "completion_tokens", "steps", "spec_draft_tokens",
                      "spec_accepted_tokens", "spec_verify_steps"):
                setattr(agg, f, getattr(agg, f) + getattr(s, f))
            agg.warming = agg.warming or s.warming
        return agg

    def replica_stats(self) -> List[EngineStats]:
        return [e.stats() for e in self.engines]

    def set_warming(self, on: bool):
        for e in self.engines:
            e.set_warming(on)

    def shutdown(self):
        for e in self.engines:
            e.shutdown()
