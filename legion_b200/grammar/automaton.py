"""Byte-level automaton for JSON constrained by a JSON Schema.

The state is an immutable tuple (a stack of frames), so trying a byte is ``step(state, byte) -> new state or
None`` and a token is tried by folding its bytes; the vocabulary mask walks a trie of the tokens' bytes with
this function. Supported schema: type object / array / string / number / integer / boolean / null, enum, const,
properties + required (+ additionalProperties false by default when properties are given), items, minItems /
maxItems, anyOf / oneOf, and the empty schema (any JSON). Whitespace: one optional space after ':' and ','.

Reference: JSON Schema -> byte-level AST -> byte NFA / lazy DFA (``src/grammar/schema.rs``, ``matcher.rs``).
"""
from __future__ import annotations

import json
from typing import Dict, List, Optional, Tuple

State = Tuple  # stack of frames, innermost last; () = document complete

_DIGITS = frozenset(b"0123456789")
_HEX = frozenset(b"0123456789abcdefABCDEF")
_ESC = frozenset(b'"\\/bfnrt')


class Schema:
    """Schemas are interned into a table so frames can refer to them by index."""

    def __init__(self, root: dict):
        self.nodes: List[dict] = []
        self.defs = root.get("$defs") or root.get("definitions") or {}
        self._any_src: dict = {}
        self.any_id = self._intern(self._any_src)
        self.root = self._intern(root)

    def _resolve(self, s):
        seen = 0
        while isinstance(s, dict) and "$ref" in s and seen < 32:
            ref = s["$ref"]
            name = ref.rsplit("/", 1)[-1]
            if name not in self.defs:
                raise ValueError(f"unresolvable $ref {ref!r}")
            s = self.defs[name]
            seen += 1
        return s

    def _intern(self, s) -> int:
        if s is True or s is None:
            s = {}
        if not isinstance(s, dict):
            raise ValueError("schema must be an object")
        s = self._resolve(s)
        for i, n in enumerate(self.nodes):
            if n.get("_src") is s:
                return i
        node: dict = {"_src": s}
        idx = len(self.nodes)
        self.nodes.append(node)
        if "const" in s:
            node["alts"] = (json.dumps(s["const"], ensure_ascii=False, separators=(",", ":")).encode(),)
        elif "enum" in s:
            if not s["enum"]:
                raise ValueError("enum must not be empty")
            node["alts"] = tuple(json.dumps(v, ensure_ascii=False, separators=(",", ":")).encode() for v in s["enum"])
        elif "anyOf" in s or "oneOf" in s:
            node["any"] = tuple(self._intern(x) for x in (s.get("anyOf") or s.get("oneOf")))
        else:
            t = s.get("type")
            if isinstance(t, list):
                node["any"] = tuple(self._intern(dict(s, type=x)) for x in t)
            elif t is None and not s.get("properties") and "items" not in s:
                node["kind"] = "any"
            else:
                t = t or ("object" if "properties" in s else "array")
                if t not in ("object", "array", "string", "number", "integer", "boolean", "null"):
                    raise ValueError(f"unsupported schema type {t!r}")
                node["kind"] = t
                if t == "object":
                    props = s.get("properties") or {}
                    node["props"] = {k: self._intern(v) for k, v in props.items()}
                    node["required"] = frozenset(s.get("required") or ())
                    ap = s.get("additionalProperties", False if props else True)
                    node["extra"] = self._intern(ap if isinstance(ap, dict) else {}) if ap is not False else None
                    unknown = node["required"] - set(props)
                    if unknown and node["extra"] is None:
                        raise ValueError(f"required properties {sorted(unknown)} are not declared")
                elif t == "array":
                    node["items"] = self._intern(s.get("items", {}))
                    node["min"] = int(s.get("minItems", 0))
                    node["max"] = int(s["maxItems"]) if "maxItems" in s else None
        return idx


ANY_KINDS = ("object", "array", "string", "number", "boolean", "null")


def start_state(schema: Schema) -> State:
    return (("val", schema.root, True),)


def is_complete(state: State) -> bool:
    """True when the document may end here (a top-level number can end without a delimiter)."""
    if state == ():
        return True
    return len(state) == 1 and state[0][0] == "num" and state[0][1] in ("int", "zero", "frac", "exp")


def _begin_value(sc: Schema, sid: int, b: int, rest: State) -> List[State]:
    """States after reading byte b as the first byte of a value of schema sid."""
    n = sc.nodes[sid]
    out: List[State] = []
    if "alts" in n:
        cands = tuple(a[1:] for a in n["alts"] if a and a[0] == b)
        if cands:
            out.append(_alts_state(cands, rest))
        return out
    if "any" in n:
        for sub in n["any"]:
            out.extend(_begin_value(sc, sub, b, rest))
        return out
    kind = n["kind"]
    kinds = ANY_KINDS if kind == "any" else (kind,)
    for k in kinds:
        if k == "object" and b == 0x7B:
            osid = sid if kind == "object" else -1
            out.append(rest + (("obj", osid, "first", frozenset()),))
        elif k == "array" and b == 0x5B:
            out.append(rest + (("arr", sid if kind == "array" else -1, "first", 0),))
        elif k == "string" and b == 0x22:
            out.append(rest + (("str", "n", 0),))
        elif k in ("number", "integer"):
            integer = k == "integer"
            if b == 0x2D:
                out.append(rest + (("num", "sign", integer),))
            elif b == 0x30:
                out.append(rest + (("num", "zero", integer),))
            elif b in _DIGITS:
                out.append(rest + (("num", "int", integer),))
        elif k == "boolean":
            if b == 0x74:
                out.append(_alts_state((b"rue",), rest))
            elif b == 0x66:
                out.append(_alts_state((b"alse",), rest))
        elif k == "null" and b == 0x6E:
            out.append(_alts_state((b"ull",), rest))
    return out


def _alts_state(cands: Tuple[bytes, ...], rest: State) -> State:
    if any(len(c) == 0 for c in cands) and len(cands) == 1:
        return rest
    return rest + (("alts", cands),)


def step(sc: Schema, state: State, b: int) -> List[State]:
    """All successor states (the automaton is an NFA because of anyOf / any); empty list = byte refused."""
    if not state:
        return []
    top, rest = state[-1], state[:-1]
    kind = top[0]
    if kind == "val":
        if b == 0x20 and len(top) == 2:           # one optional space before a value
            return [rest + (("val", top[1], True),)]
        return _begin_value(sc, top[1], b, rest)
    if kind == "alts":
        cands = tuple(c[1:] for c in top[1] if c and c[0] == b)
        out = []
        done = any(len(c) == 0 for c in cands)
        more = tuple(c for c in cands if c)
        if done:
            out.append(rest)
        if more:
            out.append(rest + (("alts", more),))
        # an alternative that is complete may also be followed by a delimiter handled by the parent
        return out
    if kind == "str":
        mode = top[1]
        if mode == "n":
            if b == 0x22:
                return [rest]
            if b == 0x5C:
                return [rest + (("str", "e", 0),)]
            if b >= 0x20:
                return [state]
            return []
        if mode == "e":
            if b == 0x75:
                return [rest + (("str", "u", 4),)]
            return [rest + (("str", "n", 0),)] if b in _ESC else []
        if mode == "u":
            if b not in _HEX:
                return []
            return [rest + (("str", "u", top[2] - 1),)] if top[2] > 1 else [rest + (("str", "n", 0),)]
    if kind == "num":
        ph, integer = top[1], top[2]
        if ph == "sign":
            if b == 0x30:
                return [rest + (("num", "zero", integer),)]
            return [rest + (("num", "int", integer),)] if b in _DIGITS else []
        if ph in ("int", "zero"):
            if ph == "int" and b in _DIGITS:
                return [state]
            if b == 0x2E and not integer:
                return [rest + (("num", "dot", integer),)]
            if b in (0x65, 0x45) and not integer:
                return [rest + (("num", "e", integer),)]
            return step(sc, rest, b)          # the number ended: the parent sees this byte
        if ph == "dot":
            return [rest + (("num", "frac", integer),)] if b in _DIGITS else []
        if ph == "frac":
            if b in _DIGITS:
                return [state]
            if b in (0x65, 0x45):
                return [rest + (("num", "e", integer),)]
            return step(sc, rest, b)
        if ph == "e":
            if b in (0x2B, 0x2D):
                return [rest + (("num", "esign", integer),)]
            return [rest + (("num", "exp", integer),)] if b in _DIGITS else []
        if ph == "esign":
            return [rest + (("num", "exp", integer),)] if b in _DIGITS else []
        if ph == "exp":
            return [state] if b in _DIGITS else step(sc, rest, b)
    if kind == "obj":
        return _step_obj(sc, top, rest, b)
    if kind == "arr":
        return _step_arr(sc, top, rest, b)
    if kind == "key":
        return _step_key(sc, top, rest, b)
    return []


def _step_obj(sc: Schema, top, rest: State, b: int) -> List[State]:
    sid, ph, seen = top[1], top[2], top[3]
    node = sc.nodes[sid] if sid >= 0 else None
    required = node["required"] if node else frozenset()
    if ph in ("first", "next"):
        if b == 0x20 and ph == "next":
            return [rest + (("obj", sid, "next_sp", seen),)]
        if b == 0x7D and ph == "first" and required <= seen:
            return [rest]
        if b == 0x22:
            return _open_key(sc, sid, seen, rest)
        return []
    if ph == "next_sp":
        return _open_key(sc, sid, seen, rest) if b == 0x22 else []
    if ph == "colon":                      # after the closing quote of a key; top = (.., seen, value sid)
        if b == 0x3A:
            return [rest + (("obj", sid, "after", seen), ("val", top[4]))]
        return []
    if ph == "after":
        more = node is None or node["extra"] is not None or any(k not in seen for k in node["props"])
        if b == 0x2C and more:
            return [rest + (("obj", sid, "next", seen),)]
        if b == 0x7D and required <= seen:
            return [rest]
        return []
    return []


def _open_key(sc: Schema, sid: int, seen, rest: State) -> List[State]:
    node = sc.nodes[sid] if sid >= 0 else None
    out: List[State] = []
    if node and node["props"]:
        cands = tuple((k.encode(), k) for k in node["props"] if k not in seen)
        if cands:
            out.append(rest + (("key", sid, seen, cands),))
    if node is None or node["extra"] is not None:
        out.append(rest + (("key", sid, seen, None),))
    return out


def _step_key(sc: Schema, top, rest: State, b: int) -> List[State]:
    _, sid, seen, cands = top
    node = sc.nodes[sid] if sid >= 0 else None
    if cands is None:                      # free key (additional property): any string without escapes
        if b == 0x22:
            vs = node["extra"] if node else sc.any_id
            return [rest + (("obj", sid, "colon", seen, vs),)]
        if b >= 0x20 and b != 0x5C:
            return [(rest + (top,))]
        return []
    out: List[State] = []
    if b == 0x22:
        for rem, name in cands:
            if not rem:
                out.append(rest + (("obj", sid, "colon", seen | {name}, node["props"][name]),))
        return out
    nxt = tuple((rem[1:], name) for rem, name in cands if rem and rem[0] == b)
    return [rest + (("key", sid, seen, nxt),)] if nxt else []


def _step_arr(sc: Schema, top, rest: State, b: int) -> List[State]:
    _, sid, ph, count = top
    node = sc.nodes[sid] if sid >= 0 else None
    items = node["items"] if node else sc.any_id
    lo = node["min"] if node else 0
    hi = node["max"] if node else None
    if ph == "first":
        if b == 0x5D:
            return [rest] if lo <= 0 else []
        if hi is not None and hi <= 0:
            return []
        return step(sc, rest + (("arr", sid, "after", 1), ("val", items, True)), b)
    if ph == "after":
        if b == 0x5D:
            return [rest] if count >= lo else []
        if b == 0x2C and (hi is None or count < hi):
            return [rest + (("arr", sid, "after", count + 1), ("val", items))]
        return []
    return []
