"""Chat template rendering with the Jinja template stored in the checkpoint, with the semantics HF
transformers gives templates: ``trim_blocks`` / ``lstrip_blocks``, ``raise_exception``, ``strftime_now``,
``tojson`` that keeps non-ASCII text, ``messages`` / ``tools`` / ``add_generation_prompt`` /
``enable_thinking`` and any ``chat_template_kwargs`` in scope (``src/chat_template.rs:41-86`` in the reference).
"""
from __future__ import annotations

import datetime
import json
from functools import lru_cache
from typing import Any, Dict, List, Optional

import jinja2
from jinja2.sandbox import ImmutableSandboxedEnvironment


class TemplateError(ValueError):
    pass


def _raise(msg):
    raise TemplateError(str(msg))


def _tojson(value, indent=None, ensure_ascii=False, separators=None, sort_keys=False):
    return json.dumps(value, ensure_ascii=ensure_ascii, indent=indent, separators=separators, sort_keys=sort_keys)


@lru_cache(maxsize=16)
def _compile(template: str):
    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True,
                                        extensions=["jinja2.ext.loopcontrols"])
    env.filters["tojson"] = _tojson
    env.globals["raise_exception"] = _raise
    env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
    return env.from_string(template)


def _msg_dict(m) -> Dict[str, Any]:
    if isinstance(m, dict):
        d = dict(m)
    else:
        d = {"role": m.role, "content": m.content}
        for k in ("tool_calls", "tool_call_id", "name", "reasoning_content"):
            v = getattr(m, k, None)
            if v is not None:
                d[k] = v
    # content parts -> text (images leave a placeholder the vision path replaces)
    if isinstance(d.get("content"), list):
        parts = []
        for p in d["content"]:
            t = p.get("type")
            if t in ("text", "input_text", "output_text"):
                parts.append(p.get("text", ""))
            elif t in ("image_url", "image", "input_image"):
                parts.append("<|vision_start|><|image_pad|><|vision_end|>")
        d["content"] = "".join(parts)
    if d.get("content") is None:
        d["content"] = ""
    if d.get("tool_calls"):
        tcs = []
        for tc in d["tool_calls"]:
            fn = dict(tc.get("function", tc))
            args = fn.get("arguments")
            if isinstance(args, str):
                try:
                    fn["arguments"] = json.loads(args)
                except ValueError:
                    pass
            tcs.append({"id": tc.get("id"), "type": "function", "function": fn})
        d["tool_calls"] = tcs
    return d


def render(template: str, messages: List[Any], tools: Optional[List[dict]] = None, add_generation_prompt: bool = True,
           bos_token: str = "", eos_token: str = "", **kwargs) -> str:
    try:
        return _compile(template).render(messages=[_msg_dict(m) for m in messages], tools=tools or None,
                                         add_generation_prompt=add_generation_prompt, bos_token=bos_token,
                                         eos_token=eos_token, **kwargs)
    except jinja2.TemplateError as e:
        raise TemplateError(f"chat template failed: {e}") from e
