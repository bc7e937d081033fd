"""Wire formats <-> engine types: OpenAI chat / completions / responses and Anthropic messages requests
become ``GenerateRequest``; validation errors become ``ApiError`` rendered in the caller API's shape.

Rules (``src/server/convert.rs:37-137,165-232`` and ``docs/api.md`` of the reference): unknown JSON fields are
ignored; temperature 0..2 (Anthropic 0..1), top_p (0,1], min_p 0..1, penalties -2..2, repetition_penalty > 0,
top_logprobs <= 20, min_tokens <= max_tokens; images only as ``data:`` URLs / base64 (png, jpeg, webp, gif);
``enable_thinking`` boolean inside ``chat_template_kwargs``; ``/v1/responses`` is stateless
(``previous_response_id`` and ``store=true`` are refused); sampling defaults resolve request > operator >
model > OpenAI.
"""
from __future__ import annotations

import base64
import re
from typing import Any, Dict, List, Optional

from ..engine.types import ChatMessage, GenerateRequest, SamplingParams


class ApiError(Exception):
    def __init__(self, status: int, message: str, kind: str = "invalid_request_error", param: Optional[str] = None):
        super().__init__(message)
        self.status, self.message, self.kind, self.param = status, message, kind, param


_IMG = re.compile(r"^data:image/(png|jpeg|jpg|webp|gif);base64,(.*)$", re.S)


def _num(d: dict, key: str, default, typ=float, param=None):
    v = d.get(key, None)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ApiError(400, f"{key} must be a number", param=param or key)
    return typ(v)


def _stop(v) -> List[str]:
    if v is None:
        return []
    if isinstance(v, str):
        return [v]
    if isinstance(v, list) and all(isinstance(s, str) for s in v):
        if len(v) > 16:
            raise ApiError(400, "at most 16 stop sequences are supported", param="stop")
        return list(v)
    raise ApiError(400, "stop must be a string or a list of strings", param="stop")


def sampling_from(body: dict, defaults: Optional[dict], default_max_tokens: int, anthropic: bool = False) -> SamplingParams:
    d = dict(defaults or {})
    max_key = "max_tokens"
    max_tokens = body.get("max_completion_tokens", body.get("max_tokens", body.get("max_output_tokens")))
    if max_tokens is None:
        if anthropic:
            raise ApiError(400, "max_tokens is required", param="max_tokens")
        max_tokens = default_max_tokens
    if isinstance(max_tokens, bool) or not isinstance(max_tokens, int) or max_tokens < 1:
        raise ApiError(400, "max_tokens must be a positive integer", param=max_key)
    n = body.get("n")
    if n is not None and (isinstance(n, bool) or n != 1):
        raise ApiError(400, "only n=1 is supported", param="n")
    lp = body.get("logprobs")
    top_lp = _num(body, "top_logprobs", 0, int)
    if isinstance(lp, int) and not isinstance(lp, bool):      # legacy completions: logprobs = N
        top_lp, lp = lp, lp > 0
    sp = SamplingParams(
        temperature=_num(body, "temperature", d.get("temperature", 1.0)),
        top_p=_num(body, "top_p", d.get("top_p", 1.0)),
        top_k=_num(body, "top_k", d.get("top_k", 0), int),
        min_p=_num(body, "min_p", d.get("min_p", 0.0)),
        presence_penalty=_num(body, "presence_penalty", d.get("presence_penalty", 0.0)),
        frequency_penalty=_num(body, "frequency_penalty", d.get("frequency_penalty", 0.0)),
        repetition_penalty=_num(body, "repetition_penalty", d.get("repetition_penalty", 1.0)),
        seed=_num(body, "seed", None, int), max_tokens=int(max_tokens), min_tokens=_num(body, "min_tokens", 0, int),
        stop=_stop(body.get("stop", body.get("stop_sequences"))),
        stop_token_ids=[int(x) for x in (body.get("stop_token_ids") or [])],
        ignore_eos=bool(body.get("ignore_eos", False)), logprobs=bool(lp), top_logprobs=top_lp,
        logit_bias={int(k): float(v) for k, v in (body.get("logit_bias") or {}).items()})
    try:
        sp.validate(anthropic=anthropic)
    except ValueError as e:
        raise ApiError(400, str(e)) from None
    return sp


def _image_bytes(url: str) -> bytes:
    m = _IMG.match(url or "")
    if not m:
        raise ApiError(400, "images must be data: URLs with base64 png, jpeg, webp or gif content", param="messages")
    try:
        return base64.b64decode(m.group(2), validate=False)
    except Exception:
        raise ApiError(400, "image is not valid base64", param="messages") from None


def _openai_message(m: dict, images: List[bytes]) -> ChatMessage:
    if not isinstance(m, dict) or "role" not in m:
        raise ApiError(400, "each message needs a role", param="messages")
    role = m["role"]
    if role == "developer":
        role = "system"
    if role not in ("system", "user", "assistant", "tool"):
        raise ApiError(400, f"unknown message role {role!r}", param="messages")
    content = m.get("content")
    if isinstance(content, list):
        parts = []
        for p in content:
            t = p.get("type")
            if t in ("text", "input_text", "output_text"):
                parts.append({"type": "text", "text": p.get("text", "")})
            elif t == "image_url":
                url = p.get("image_url", {})
                url = url.get("url") if isinstance(url, dict) else url
                images.append(_image_bytes(url))
                parts.append({"type": "image"})
            elif t == "input_image":
                images.append(_image_bytes(p.get("image_url")))
                parts.append({"type": "image"})
            else:
                raise ApiError(400, f"unsupported content part type {t!r}", param="messages")
        content = parts
    elif content is None:
        content = ""
    elif not isinstance(content, str):
        raise ApiError(400, "message content must be a string or a list of parts", param="messages")
    return ChatMessage(role=role, content=content, tool_calls=m.get("tool_calls"), tool_call_id=m.get("tool_call_id"),
                       name=m.get("name"), reasoning_content=m.get("reasoning_content"))


def _thinking(body: dict) -> Optional[bool]:
    kw = body.get("chat_template_kwargs") or {}
    if "enable_thinking" in kw:
        if not isinstance(kw["enable_thinking"], bool):
            raise ApiError(400, "chat_template_kwargs.enable_thinking must be a boolean")
        return kw["enable_thinking"]
    return None


def _tools(body: dict) -> Optional[List[dict]]:
    tools = body.get("tools")
    if not tools:
        return None
    out = []
    for t in tools:
        if t.get("type", "function") != "function":
            continue
        fn = t.get("function") or {k: t[k] for k in ("name", "description", "parameters") if k in t}
        if "name" not in fn:
            raise ApiError(400, "each tool needs a function name", param="tools")
        out.append({"type": "function", "function": fn})
    if body.get("tool_choice") == "none":
        return None
    return out or None


def chat_request(body: dict, defaults=None, default_max_tokens: int = 4096) -> GenerateRequest:
    msgs = body.get("messages")
    if not isinstance(msgs, list) or not msgs:
        raise ApiError(400, "messages must be a non-empty list", param="messages")
    images: List[bytes] = []
    messages = [_openai_message(m, images) for m in msgs]
    rf = body.get("response_format")
    if rf is not None and (not isinstance(rf, dict) or rf.get("type") not in ("text", "json_object", "json_schema")):
        raise ApiError(400, "response_format.type must be text, json_object or json_schema", param="response_format")
    return GenerateRequest(model=body.get("model", ""), messages=messages,
                           sampling=sampling_from(body, defaults, default_max_tokens), tools=_tools(body),
                           tool_choice=body.get("tool_choice"), response_format=rf, enable_thinking=_thinking(body),
                           images=images, priority=int(body.get("priority", 0) or 0))


def completion_request(body: dict, defaults=None, default_max_tokens: int = 16) -> GenerateRequest:
    prompt = body.get("prompt")
    tokens = None
    if isinstance(prompt, list):
        if prompt and all(isinstance(x, int) for x in prompt):
            tokens, prompt = list(prompt), None
        elif len(prompt) == 1 and isinstance(prompt[0], str):
            prompt = prompt[0]
        else:
            raise ApiError(400, "prompt must be a string or a list of token ids", param="prompt")
    elif not isinstance(prompt, str):
        raise ApiError(400, "prompt is required", param="prompt")
    return GenerateRequest(model=body.get("model", ""), prompt=prompt, prompt_tokens=tokens,
                           sampling=sampling_from(body, defaults, default_max_tokens), echo=bool(body.get("echo", False)),
                           priority=int(body.get("priority", 0) or 0))


def anthropic_request(body: dict, defaults=None) -> GenerateRequest:
    msgs = body.get("messages")
    if not isinstance(msgs, list) or not msgs:
        raise ApiError(400, "messages must be a non-empty list", param="messages")
    images: List[bytes] = []
    out: List[ChatMessage] = []
    system = body.get("system")
    if system:
        if isinstance(system, list):
            system = "".join(p.get("text", "") for p in system)
        out.append(ChatMessage(role="system", content=system))
    for m in msgs:
        role = m.get("role")
        if role not in ("user", "assistant"):
            raise ApiError(400, f"unknown message role {role!r}", param="messages")
        content = m.get("content")
        if isinstance(content, str):
            out.append(ChatMessage(role=role, content=content))
            continue
        text_parts, tool_calls = [], []
        for p in content or []:
            t = p.get("type")
            if t == "text":
                text_parts.append({"type": "text", "text": p.get("text", "")})
            elif t == "image":
                src = p.get("source", {})
                if src.get("type") != "base64":
                    raise ApiError(400, "images must be base64 sources", param="messages")
                images.append(base64.b64decode(src.get("data", "")))
                text_parts.append({"type": "image"})
            elif t == "tool_use":
                tool_calls.append({"id": p.get("id"), "type": "function",
                                   "function": {"name": p.get("name"), "arguments": p.get("input", {})}})
            elif t == "tool_result":
                c = p.get("content")
                if isinstance(c, list):
                    c = "".join(x.get("text", "") for x in c)
                out.append(ChatMessage(role="tool", content=c or "", tool_call_id=p.get("tool_use_id")))
            elif t == "thinking":
                continue
            else:
                raise ApiError(400, f"unsupported content block type {t!r}", param="messages")
        if text_parts or tool_calls:
            out.append(ChatMessage(role=role, content=text_parts, tool_calls=tool_calls or None))
    tools = None
    if body.get("tools"):
        tools = [{"type": "function", "function": {"name": t["name"], "description": t.get("description", ""),
                                                   "parameters": t.get("input_schema", {})}} for t in body["tools"]]
    thinking = body.get("thinking")
    enable = None
    if isinstance(thinking, dict):
        enable = thinking.get("type") == "enabled"
    return GenerateRequest(model=body.get("model", ""), messages=out,
                           sampling=sampling_from(body, defaults, 0, anthropic=True), tools=tools,
                           enable_thinking=enable, images=images)


def responses_request(body: dict, defaults=None, default_max_tokens: int = 4096) -> GenerateRequest:
    if body.get("previous_response_id"):
        raise ApiError(400, "previous_response_id is not supported: the responses endpoint is stateless",
                       param="previous_response_id")
    if body.get("store") is True:
        raise ApiError(400, "store=true is not supported: responses are not kept", param="store")
    inp = body.get("input")
    msgs: List[dict] = []
    if body.get("instructions"):
        msgs.append({"role": "system", "content": body["instructions"]})
    if isinstance(inp, str):
        msgs.append({"role": "user", "content": inp})
    elif isinstance(inp, list):
        for item in inp:
            t = item.get("type", "message")
            if t == "message":
                msgs.append({"role": item.get("role", "user"), "content": item.get("content", "")})
            elif t == "function_call":
                msgs.append({"role": "assistant", "content": "", "tool_calls": [
                    {"id": item.get("call_id"), "type": "function",
                     "function": {"name": item.get("name"), "arguments": item.get("arguments", "{}")}}]})
            elif t == "function_call_output":
                msgs.append({"role": "tool", "content": item.get("output", ""), "tool_call_id": item.get("call_id")})
    else:
        raise ApiError(400, "input must be a string or a list of items", param="input")
    b = dict(body)
    b["messages"] = msgs
    text = body.get("text") or {}
    fmt = text.get("format") if isinstance(text, dict) else None
    if isinstance(fmt, dict) and fmt.get("type") == "json_schema":
        b["response_format"] = {"type": "json_schema", "json_schema": {"name": fmt.get("name", "out"),
                                                                       "schema": fmt.get("schema", {})}}
    elif isinstance(fmt, dict) and fmt.get("type") == "json_object":
        b["response_format"] = {"type": "json_object"}
    if body.get("reasoning") and isinstance(body["reasoning"], dict):
        b.setdefault("chat_template_kwargs", {})
    return chat_request(b, defaults, default_max_tokens)
