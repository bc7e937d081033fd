"""Token-level constraint: walks a trie of the vocabulary's byte strings with the JSON automaton to get the
set of tokens that keep the output valid (a boolean mask over the vocabulary), and advances with each
sampled token. Sub-tries made only of bytes that are always legal inside a JSON string are accepted in one
step while the automaton is inside a free string, which keeps the walk small for large vocabularies.

Reference: per-step vocabulary bitmask computed beside the forward pass, 64-entry LRU of compiled grammars
(``src/grammar/matcher.rs``, ``src/engine/lm/response_format.rs``).
"""
from __future__ import annotations

import json
from collections import OrderedDict
from typing import Dict, List, Optional, Tuple

import torch

from .automaton import Schema, is_complete, start_state, step


class _Trie:
    __slots__ = ("children", "tokens", "plain", "all_tokens")

    def __init__(self):
        self.children: Dict[int, "_Trie"] = {}
        self.tokens: List[int] = []
        self.plain = True          # every byte below this node is legal inside a JSON string as is
        self.all_tokens: Optional[List[int]] = None


def _plain_byte(b: int) -> bool:
    return b >= 0x20 and b not in (0x22, 0x5C)


class TokenTrie:
    def __init__(self, tokenizer):
        self.root = _Trie()
        self.vocab = tokenizer.vocab_size
        special = set(getattr(tokenizer, "_special_ids", ()) or ())
        special |= set(getattr(tokenizer, "_sp_inv", {}).keys())
        for tid in range(tokenizer.vocab_size):
            if tid in special:
                continue
            try:
                bs = tokenizer.token_bytes(tid)
            except Exception:
                continue
            if not bs or bs.startswith(b"<0x"):
                continue
            node = self.root
            for b in bs:
                nxt = node.children.get(b)
                if nxt is None:
                    nxt = node.children[b] = _Trie()
                node = nxt
            node.tokens.append(tid)
        self._finish(self.root)

    def _finish(self, node: _Trie) -> List[int]:
        allt = list(node.tokens)
        plain = True
        for b, ch in node.children.items():
            allt.extend(self._finish(ch))
            plain = plain and ch.plain and _plain_byte(b)
        node.plain = plain
        node.all_tokens = allt
        return allt


_tries: Dict[int, TokenTrie] = {}


def trie_for(tokenizer) -> TokenTrie:
    t = _tries.get(id(tokenizer))
    if t is None:
        t = _tries[id(tokenizer)] = TokenTrie(tokenizer)
    return t


class Matcher:
    """The engine-facing constraint object: ``mask()``, ``advance(token)``, ``finished()``."""

    def __init__(self, schema: Schema, tokenizer):
        self.schema = schema
        self.tok = tokenizer
        self.trie = trie_for(tokenizer)
        self.states = [start_state(schema)]
        self.eos = tuple(tokenizer.eos_ids)
        self._mask_cache: Optional[torch.Tensor] = None

    def clone(self) -> "Matcher":
        m = Matcher.__new__(Matcher)
        m.schema, m.tok, m.trie, m.eos = self.schema, self.tok, self.trie, self.eos
        m.states = list(self.states)
        m._mask_cache = None
        return m

    def finished(self) -> bool:
        return all(s == () for s in self.states) and bool(self.states)

    def can_end(self) -> bool:
        return any(is_complete(s) for s in self.states)

    def _in_free_string(self, states) -> bool:
        return all(s and s[-1][0] == "str" and s[-1][1] == "n" for s in states)

    def mask(self) -> torch.Tensor:
        if self._mask_cache is not None:
            return self._mask_cache
        allowed = torch.zeros(self.trie.vocab, dtype=torch.bool)
        ids: List[int] = []
        sc = self.schema

        def walk(node: _Trie, states):
            for b, ch in node.children.items():
                if ch.plain and _plain_byte(b) and self._in_free_string(states):
                    ids.extend(ch.all_tokens)
                    continue
                nxt = []
                for st in states:
                    nxt.extend(step(sc, st, b))
                if not nxt:
                    continue
                nxt = list(dict.fromkeys(nxt))
                ids.extend(ch.tokens)
                if ch.children:
                    walk(ch, nxt)

        live = [s for s in self.states if s != ()]
        if live:
            walk(self.trie.root, live)
        if ids:
            allowed[torch.tensor(ids, dtype=torch.long)] = True
        if self.can_end():
            for e in self.eos:
                if 0 <= e < self.trie.vocab:
                    allowed[e] = True
        if not bool(allowed.any()):          # dead end (should not happen): let the sequence stop
            for e in self.eos:
                allowed[e] = True
        self._mask_cache = allowed
        return allowed

    def advance(self, token: int):
        self._mask_cache = None
        if token in self.eos:
            self.states = [()]
            return
        try:
            bs = self.tok.token_bytes(token)
        except Exception:
            bs = b""
        states = self.states
        for b in bs:
            nxt = []
            for st in states:
                nxt.extend(step(self.schema, st, b))
            states = list(dict.fromkeys(nxt))
            if not states:
                break
        self.states = states or [()]

    def accepts(self, text: str) -> bool:
        """Whole-document check (tests and tools)."""
        states = [start_state(self.schema)]
        for b in text.encode():
            nxt = []
            for st in states:
                nxt.extend(step(self.schema, st, b))
            states = list(dict.fromkeys(nxt))
            if not states:
                return False
        return any(is_complete(s) for s in states)


_compiled: "OrderedDict[str, Schema]" = OrderedDict()
_LRU = 64


def compile_schema(schema: dict) -> Schema:
    key = json.dumps(schema, sort_keys=True)
    sc = _compiled.get(key)
    if sc is None:
        sc = Schema(schema)
        _compiled[key] = sc
        while len(_compiled) > _LRU:
            _compiled.popitem(last=False)
    else:
        _compiled.move_to_end(key)
    return sc


def compile_response_format(fmt: dict, tokenizer) -> Optional[Matcher]:
    """``{"type": "json_object"}`` or ``{"type": "json_schema", "json_schema": {"schema": {...}}}`` -> Matcher.
    Raises ValueError for schemas outside the supported subset."""
    t = fmt.get("type")
    if t in (None, "text"):
        return None
    if t == "json_object":
        return Matcher(compile_schema({"type": "object", "additionalProperties": True}), tokenizer)
    if t == "json_schema":
        js = fmt.get("json_schema") or {}
        schema = js.get("schema", js if "type" in js or "properties" in js else None)
        if schema is None:
            raise ValueError("json_schema needs a schema")
        return Matcher(compile_schema(schema), tokenizer)
    raise ValueError(f"unsupported response_format type {t!r}")
