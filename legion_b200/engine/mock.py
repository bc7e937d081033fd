"""A GPU-free engine for the HTTP layer's tests and for ``legion serve`` without a model.

Behaviour (``src/engine/mock.rs:1-60`` in the reference): the reply echoes the last user message word by
word; a message of the form ``/tool name {json}`` produces a scripted tool call; ``ignore_eos`` keeps
emitting filler tokens up to ``max_tokens``; log-probabilities are synthetic; a request over
``max_waiting`` concurrent requests is refused as overloaded.
"""
from __future__ import annotations

import json
import threading
import time
import uuid
from typing import List, Optional

from .types import (CancelToken, ChatMessage, Engine, EngineOverloaded, EngineStats, FinishReason, GenerateRequest,
                    TokenEvent, TokenLogprob, TokenStream, Usage)


class MockEngine(Engine):
    def __init__(self, model_name: str = "mock", delay_s: float = 0.0, max_in_flight: int = 1024):
        self.model_name = model_name
        self.delay_s = delay_s
        self.max_in_flight = max_in_flight
        self._in_flight = 0
        self._lock = threading.Lock()
        self._stats = EngineStats()
        self._warming = False

    def models(self):
        return [{"id": self.model_name, "object": "model", "owned_by": "legion-b200", "context_length": 8192}]

    def _text_of(self, req: GenerateRequest) -> str:
        if req.messages:
            for m in reversed(req.messages):
                if m.role == "user":
                    if isinstance(m.content, list):
                        return "".join(p.get("text", "") for p in m.content if isinstance(p, dict))
                    return m.content or ""
            return ""
        return req.prompt or ""

    def count_tokens(self, req: GenerateRequest) -> int:
        n = 0
        for m in (req.messages or []):
            c = m.content if isinstance(m.content, str) else " ".join(p.get("text", "") for p in m.content)
            n += len(c.split()) + 3
        return n + len((req.prompt or "").split())

    def check_response_format(self, fmt):
        if fmt and fmt.get("type") == "json_schema" and "json_schema" not in fmt:
            raise ValueError("response_format json_schema needs a schema")

    def set_warming(self, on: bool):
        self._warming = on

    def stats(self) -> EngineStats:
        self._stats.running = self._in_flight
        self._stats.warming = self._warming
        return self._stats

    def generate(self, req: GenerateRequest) -> TokenStream:
        req.sampling.validate()
        with self._lock:
            if self._in_flight >= self.max_in_flight:
                raise EngineOverloaded("too many requests in flight")
            self._in_flight += 1
        stream = TokenStream(CancelToken())
        t = threading.Thread(target=self._run, args=(req, stream), daemon=True)
        t.start()
        return stream

    def _run(self, req: GenerateRequest, stream: TokenStream):
        try:
            text = self._text_of(req)
            n_prompt = self.count_tokens(req)
            usage = Usage(prompt_tokens=n_prompt)
            stream.put(TokenEvent(kind="started", prompt_tokens=n_prompt))
            sp = req.sampling
            reason = FinishReason.STOP
            if text.startswith("/tool ") and req.tools:
                _, name, *rest = text.split(" ", 2)
                args = rest[0] if rest else "{}"
                try:
                    json.loads(args)
                except ValueError:
                    args = json.dumps({"input": args})
                stream.put(TokenEvent(kind="tool_call", tool_call={"id": "call_" + uuid.uuid4().hex[:24], "name": name,
                                                                   "arguments": args}))
                usage.completion_tokens = 1
                reason = FinishReason.TOOL_CALLS
            else:
                words = text.split(" ") if text else ["ok"]
                pieces = [w if i == 0 else " " + w for i, w in enumerate(words)]
                if req.response_format and req.response_format.get("type") in ("json_object", "json_schema"):
                    pieces = ["{", '"echo"', ":", json.dumps(text), "}"]
                if sp.ignore_eos:
                    while len(pieces) < sp.max_tokens:
                        pieces.append(" filler")
                emitted = ""
                for i, p in enumerate(pieces):
                    if stream.cancel_token.cancelled:
                        reason = FinishReason.CANCELLED
                        break
                    if i >= sp.max_tokens:
                        reason = FinishReason.LENGTH
                        break
                    hit = next((s for s in sp.stop if s and s in emitted + p), None)
                    if hit is not None:
                        cut = (emitted + p).index(hit) - len(emitted)
                        if cut > 0:
                            stream.put(TokenEvent(kind="text", text=p[:cut], token_ids=[i]))
                        reason = FinishReason.STOP_SEQUENCE
                        break
                    lps: List[TokenLogprob] = []
                    if sp.logprobs:
                        lps = [TokenLogprob(p, i, -0.1, [TokenLogprob(p, i, -0.1)] * min(1, sp.top_logprobs))]
                    stream.put(TokenEvent(kind="text", text=p, token_ids=[i], logprobs=lps))
                    emitted += p
                    usage.completion_tokens += 1
                    if self.delay_s:
                        time.sleep(self.delay_s)
            self._stats.prompt_tokens += n_prompt
            self._stats.completion_tokens += usage.completion_tokens
            stream.put(TokenEvent(kind="finished", finish_reason=reason, usage=usage))
        except Exception as e:  # pragma: no cover
            stream.put(TokenEvent(kind="error", error=str(e)))
        finally:
            with self._lock:
                self._in_flight -= 1
