"""Strict tool calls: a schema that only admits ``{"name": <one of the tools>, "arguments": <that tool's
parameters>}`` (the hermes body between ``<tool_call>`` tags), so a constrained request cannot produce a call
the caller's tools cannot parse (``src/grammar/tool_call.rs`` in the reference)."""
from __future__ import annotations

from typing import List


def tool_call_schema(tools: List[dict]) -> dict:
    alts = []
    for t in tools:
        fn = t.get("function", t)
        params = fn.get("parameters") or {"type": "object", "additionalProperties": True}
        alts.append({"type": "object", "properties": {"name": {"const": fn["name"]}, "arguments": params},
                     "required": ["name", "arguments"]})
    if not alts:
        raise ValueError("no tools")
    return alts[0] if len(alts) == 1 else {"anyOf": alts}
