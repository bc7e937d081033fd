"""Speculative decoding: drafters, acceptance, depth policy.

Drafters propose tokens that the target verifies in ONE step: a decoding sequence feeds ``[last, d1..dk]``,
the target returns k + 1 rows, the longest agreeing prefix plus one bonus token is kept (greedy), or each
draft is accepted by exact rejection sampling (sampled requests). KV rollback is a length change;
recurrent layers do not advance during verify and replay the kept tokens afterwards
(``models.decoder.Decoder.commit_replay``). Reference design: ``src/spec/mod.rs:1-330``.

  ngram    prompt-lookup: continue the longest recent n-gram match in the sequence itself
  suffix   suffix index over the sequence plus a cross-request cache of finished replies
  mtp      the model's own next-token-prediction head, chained k times
  mtp_ngram  the same, with a prompt-lookup shortcut for sequences whose tail occurred before
  draft    a smaller model with the same vocabulary, run k times
  eagle3   one decoder layer over [embed ; fc(target layers lo/mid/hi)] with its own KV, chained
  dflash   block drafter: one pass proposes a whole block from the target's last hidden row
"""
from __future__ import annotations

from .drafters import (DflashDrafter, DraftModelDrafter, Eagle3Drafter, MtpDrafter, MtpNgramDrafter, NgramDrafter,
                       SuffixDrafter)


def make_drafter(kind: str, engine, **kw):
    if kind == "ngram":
        return NgramDrafter(engine.cfg.spec_ngram_min, engine.cfg.spec_ngram_max)
    if kind == "suffix":
        return SuffixDrafter()
    if kind == "mtp":
        return MtpDrafter(engine)
    if kind == "mtp_ngram":
        return MtpNgramDrafter(engine, engine.cfg.spec_ngram_min, engine.cfg.spec_ngram_max)
    if kind == "draft":
        return DraftModelDrafter(engine, **kw)
    if kind == "eagle3":
        return Eagle3Drafter(engine, **kw)
    if kind == "dflash":
        return DflashDrafter(engine, **kw)
    raise ValueError(f"unknown drafter {kind!r}")
