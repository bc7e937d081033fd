"""Text-side post-processing of a token stream: incremental detokenisation, stop strings with
hold-back, the ``<think>`` reasoning splitter and tool-call parsers.

Reference counterparts: ``src/engine/stop.rs`` (stop-string hold-back), ``src/engine/reasoning.rs``,
``src/engine/tool_parser.rs`` (hermes / qwen3-coder formats).
"""
from __future__ import annotations

import json
import re
import uuid
from typing import Callable, List, Optional, Tuple


class IncrementalDetokenizer:
    """Turns token ids into text without emitting half a UTF-8 character."""

    def __init__(self, decode: Callable[[List[int]], str]):
        self._decode = decode
        self._ids: List[int] = []
        self._emitted = 0        # characters of decode(self._ids) already returned
        self._prefix_ids = 0     # ids folded into the stable prefix

    def push(self, token_id: int) -> str:
        self._ids.append(token_id)
        text = self._decode(self._ids[self._prefix_ids:])
        if text.endswith("�"):
            return ""            # incomplete multi-byte character: wait for the next token
        out = text[self._emitted:]
        # fold everything but a short tail into the prefix so decode stays O(1) per token
        if len(self._ids) - self._prefix_ids > 16:
            self._prefix_ids = len(self._ids) - 4
            self._emitted = len(self._decode(self._ids[self._prefix_ids:]))
        else:
            self._emitted = len(text)
        return out


class StopChecker:
    """Holds back text that could be the beginning of a stop string."""

    def __init__(self, stops: List[str]):
        self.stops = [s for s in stops if s]
        self._held = ""
        self.hit: Optional[str] = None

    def push(self, text: str) -> str:
        if not self.stops:
            return text
        buf = self._held + text
        best = -1
        for s in self.stops:
            i = buf.find(s)
            if i >= 0 and (best < 0 or i < best):
                best, self.hit = i, s
        if best >= 0:
            self._held = ""
            return buf[:best]
        hold = 0
        for s in self.stops:
            for n in range(min(len(s) - 1, len(buf)), 0, -1):
                if buf.endswith(s[:n]):
                    hold = max(hold, n)
                    break
        self._held = buf[len(buf) - hold:] if hold else ""
        return buf[:len(buf) - hold] if hold else buf

    def flush(self) -> str:
        out, self._held = self._held, ""
        return out


class ReasoningSplitter:
    """Routes text between the reasoning markers (``<think>`` ... ``</think>`` unless others are given) to the
    reasoning channel."""

    OPEN, CLOSE = "<think>", "</think>"

    def __init__(self, starts_in_reasoning: bool = False, tags: Optional[Tuple[str, str]] = None):
        self.in_reasoning = starts_in_reasoning
        self._held = ""
        if tags:
            self.OPEN, self.CLOSE = tags

    def push(self, text: str) -> List[Tuple[str, str]]:
        """Returns [(channel, text)] with channel in {"reasoning", "text"}."""
        out: List[Tuple[str, str]] = []
        buf = self._held + text
        self._held = ""
        while buf:
            tag = self.CLOSE if self.in_reasoning else self.OPEN
            i = buf.find(tag)
            if i >= 0:
                if i:
                    out.append(("reasoning" if self.in_reasoning else "text", buf[:i]))
                buf = buf[i + len(tag):]
                self.in_reasoning = not self.in_reasoning
                if not self.in_reasoning:
                    buf = buf.lstrip("\n")
                continue
            hold = 0
            for n in range(min(len(tag) - 1, len(buf)), 0, -1):
                if buf.endswith(tag[:n]):
                    hold = n
                    break
            emit = buf[:len(buf) - hold] if hold else buf
            if emit:
                out.append(("reasoning" if self.in_reasoning else "text", emit))
            self._held = buf[len(buf) - hold:] if hold else ""
            break
        return out

    def flush(self) -> List[Tuple[str, str]]:
        if not self._held:
            return []
        out = [("reasoning" if self.in_reasoning else "text", self._held)]
        self._held = ""
        return out


class ChatFormat:
    """Output conventions of a chat model, read once from its vocabulary rather than from the architecture name (a
    checkpoint ships whatever template and tokenizer it likes; the reference's ``src/engine/lm/chat_format.rs``):

    - Gemma 4 (``<|channel>``, ``<channel|>`` and ``<|tool_call>`` are tokens): reasoning sits between
      ``<|channel>thought`` and ``<channel|>``, the model opens that channel itself, so a reply starts inside it only
      when the prompt ends with the opener; tool calls in Gemma's notation;
    - GLM 4.5 and later (``<tool_call>``, ``<arg_key>``, ``<arg_value>``): key / value tool calls;
    - otherwise ``<think>`` ... ``</think>`` when ``<think>`` is a token (a reply starts inside when the prompt's last
      opener comes after its last closer) and the configured tool-call format.

    ``stop_ids``: end-of-turn tokens beyond the tokenizer's own (``<|im_end|>``, ``<|endoftext|>``, ``<turn|>``, and
    the openers of a tool's turn ``<|tool_response>`` / ``<|observation|>``, which hand control to the caller)."""
    STOPS = ("<|im_end|>", "<|endoftext|>", "<turn|>", "<|tool_response>", "<|observation|>")

    def __init__(self, tok, tool_format: str = "hermes"):
        tid = getattr(tok, "token_to_id", None) or (lambda t: None)
        have = lambda names: all(tid(n) is not None for n in names)       # noqa: E731
        self.kind = "plain"
        self.tool_format = tool_format
        self.tags: Optional[Tuple[str, str]] = None
        self.prompt_mode = "off"
        if have(("<|channel>", "<channel|>", "<|tool_call>")):
            self.kind, self.tool_format = "gemma4", "gemma4"
            self.tags, self.prompt_mode = ("<|channel>thought", "<channel|>"), "open_at_end"
        else:
            if have(("<tool_call>", "<arg_key>", "<arg_value>")):
                self.kind, self.tool_format = "glm", "glm"
            if tid("<think>") is not None:
                self.prompt_mode = "from_prompt"
        self.stop_ids = tuple(i for i in (tid(t) for t in self.STOPS) if i is not None)

    def starts_in_reasoning(self, prompt_tail: str) -> bool:
        """Whether the reply begins inside the reasoning span, given the end of the rendered prompt."""
        o, c = self.tags or (ReasoningSplitter.OPEN, ReasoningSplitter.CLOSE)
        if self.prompt_mode == "open_at_end":
            return prompt_tail.rstrip().endswith(o)
        if self.prompt_mode == "from_prompt":
            return prompt_tail.rfind(o) > prompt_tail.rfind(c)
        return False

    def splitter(self, prompt_tail: str = "") -> ReasoningSplitter:
        return ReasoningSplitter(self.starts_in_reasoning(prompt_tail), self.tags)


_GEMMA_QUOTE = '<|"|>'


def _gemma_value(s: str):
    """One value of Gemma 4's argument notation at the head of ``s`` -> (python value, rest of the text)."""
    s = s.lstrip()
    if s.startswith(_GEMMA_QUOTE):
        j = s.find(_GEMMA_QUOTE, len(_GEMMA_QUOTE))
        if j < 0:
            raise ValueError("unterminated string")
        return s[len(_GEMMA_QUOTE):j], s[j + len(_GEMMA_QUOTE):]
    if s.startswith("{"):
        out, s = {}, s[1:].lstrip()
        while not s.startswith("}"):
            m = re.match(r"([A-Za-z_][A-Za-z0-9_\-]*)\s*:", s)
            if not m:
                raise ValueError("expected a key")
            v, s = _gemma_value(s[m.end():])
            out[m.group(1)] = v
            s = s.lstrip()
            if s.startswith(","):
                s = s[1:].lstrip()
            elif not s.startswith("}"):
                raise ValueError("expected , or }")
        return out, s[1:]
    if s.startswith("["):
        out, s = [], s[1:].lstrip()
        while not s.startswith("]"):
            v, s = _gemma_value(s)
            out.append(v)
            s = s.lstrip()
            if s.startswith(","):
                s = s[1:].lstrip()
            elif not s.startswith("]"):
                raise ValueError("expected , or ]")
        return out, s[1:]
    m = re.match(r"-?\d+(\.\d+)?([eE][+-]?\d+)?|true|false|null", s)
    if not m:
        raise ValueError("unknown value")
    return json.loads(m.group(0)), s[m.end():]


class ToolCallParser:
    """Extracts tool calls from generated text.

    ``hermes``:       <tool_call>{"name": ..., "arguments": {...}}</tool_call>
    ``qwen3_coder``:  <tool_call><function=name><parameter=key>value</parameter>...</function></tool_call>
    ``glm``:          <tool_call>name<arg_key>key</arg_key><arg_value>value</arg_value>...</tool_call> (GLM-4.5 and
                      later; a value is JSON when it parses as JSON, else the string as written)
    ``gemma4``:       <|tool_call>call:name{key:value,...}<tool_call|> in Gemma's own notation: bare keys, strings
                      wrapped in <|"|>, numbers / true / false / null, lists and nested objects as in JSON
    Text outside the tags streams through; text inside is buffered until the closing tag. The reference's parsers
    are ``src/engine/tool_parser.rs`` and ``tool_parser/{glm,gemma4}.rs``.
    """

    OPEN, CLOSE = "<tool_call>", "</tool_call>"

    def __init__(self, fmt: str = "hermes"):
        self.fmt = fmt
        if fmt == "gemma4":
            self.OPEN, self.CLOSE = "<|tool_call>", "<tool_call|>"
        self._buf = ""
        self._inside = False
        self.calls: List[dict] = []

    def push(self, text: str) -> Tuple[str, List[dict]]:
        out_text, new_calls = "", []
        buf = self._buf + text
        self._buf = ""
        while buf:
            if not self._inside:
                i = buf.find(self.OPEN)
                if i >= 0:
                    out_text += buf[:i]
                    buf = buf[i + len(self.OPEN):]
                    self._inside = True
                    continue
                hold = 0
                for n in range(min(len(self.OPEN) - 1, len(buf)), 0, -1):
                    if buf.endswith(self.OPEN[:n]):
                        hold = n
                        break
                out_text += buf[:len(buf) - hold] if hold else buf
                self._buf = buf[len(buf) - hold:] if hold else ""
                break
            j = buf.find(self.CLOSE)
            if j < 0:
                self._buf = buf
                break
            call = self._parse(buf[:j])
            if call is not None:
                new_calls.append(call)
                self.calls.append(call)
            buf = buf[j + len(self.CLOSE):]
            self._inside = False
        return out_text, new_calls

    def flush(self) -> Tuple[str, List[dict]]:
        if self._inside:
            call = self._parse(self._buf)
            self._buf, self._inside = "", False
            if call is not None:
                self.calls.append(call)
                return "", [call]
            return "", []
        out, self._buf = self._buf, ""
        return out, []

    def _parse(self, body: str) -> Optional[dict]:
        body = body.strip()
        name, args = None, None
        if self.fmt == "glm":
            i = body.find("<arg_key>")
            name = (body if i < 0 else body[:i]).strip()
            if not name or any(c in name for c in "<>\n"):
                return None
            args = {}
            for pm in re.finditer(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", body[i:] if i >= 0 else "", re.S):
                val = pm.group(2).strip("\n")
                try:
                    args[pm.group(1).strip()] = json.loads(val)
                except (ValueError, TypeError):
                    args[pm.group(1).strip()] = val
        elif self.fmt == "gemma4":
            if not body.startswith("call:") or "{" not in body:
                return None
            name = body[5:body.index("{")].strip()
            try:
                args, rest = _gemma_value(body[body.index("{"):])
            except ValueError:
                return None
            if not name or rest.strip() or not isinstance(args, dict):
                return None
        elif self.fmt == "qwen3_coder" or body.startswith("<function="):
            m = re.match(r"<function=([^>\s]+)>(.*?)(</function>)?\s*$", body, re.S)
            if not m:
                return None
            name = m.group(1)
            args = {}
            for pm in re.finditer(r"<parameter=([^>\s]+)>(.*?)</parameter>", m.group(2), re.S):
                val = pm.group(2).strip("\n")
                try:
                    args[pm.group(1)] = json.loads(val)
                except (ValueError, TypeError):
                    args[pm.group(1)] = val
        else:
            try:
                obj = json.loads(body)
            except ValueError:
                return None
            if not isinstance(obj, dict) or "name" not in obj:
                return None
            name = obj["name"]
            args = obj.get("arguments", obj.get("parameters", {}))
            if isinstance(args, str):
                try:
                    args = json.loads(args)
                except ValueError:
                    pass
        return {"id": "call_" + uuid.uuid4().hex[:24], "name": name,
                "arguments": json.dumps(args, ensure_ascii=False) if not isinstance(args, str) else args}
