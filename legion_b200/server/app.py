"""HTTP server: OpenAI- and Anthropic-compatible routes over an ``Engine``.

Routes (``docs/serving.md:540-557`` of the reference): ``GET /`` (web UI), ``/health``, ``/metrics``,
``/v1/models``, ``/models``, ``/v1/models/{id}``, ``POST /v1/chat/completions``, ``/v1/completions``,
``/v1/messages``, ``/v1/messages/count_tokens``, ``/v1/responses``, ``GET /v1/stats``, ``/v1/stats/stream``,
``/v1/logs/stream``. Middleware: request id, API key (``Authorization: Bearer`` or ``x-api-key``), body size
limit, CORS, in-flight gauge, request metrics. Errors are rendered in the shape of the API that was called;
an overloaded engine answers 429 (OpenAI) or 529 (Anthropic). A client that disconnects cancels its request.
"""
from __future__ import annotations

import asyncio
import json
import logging
import os
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, AsyncIterator, Dict, List, Optional

from fastapi import FastAPI, Request
from fastapi.responses import HTMLResponse, JSONResponse, PlainTextResponse, StreamingResponse

from .. import __version__
from ..engine.types import (Completion, Engine, EngineOverloaded, FinishReason, GenerateRequest, KvOverflow, TokenEvent,
                            Usage)
from . import convert
from .convert import ApiError
from .metrics import LogRing, Metrics

log = logging.getLogger("legion.server")


@dataclass
class ServerConfig:
    api_keys: List[str] = field(default_factory=list)
    max_request_mb: int = 64
    cors: bool = True
    default_max_tokens: int = 4096
    sampling_defaults: Dict[str, Any] = field(default_factory=dict)
    model_aliases: Dict[str, str] = field(default_factory=dict)
    shutdown_timeout_s: float = 30.0
    fair_share: bool = False


def _openai_error(status: int, message: str, kind: str = "invalid_request_error", param=None) -> JSONResponse:
    return JSONResponse({"error": {"message": message, "type": kind, "param": param, "code": None}}, status_code=status)


def _anthropic_error(status: int, message: str, kind: str = "invalid_request_error") -> JSONResponse:
    return JSONResponse({"type": "error", "error": {"type": kind, "message": message}}, status_code=status)


def _finish_openai(r: Optional[FinishReason]) -> str:
    return {FinishReason.STOP: "stop", FinishReason.STOP_SEQUENCE: "stop", FinishReason.LENGTH: "length",
            FinishReason.TOOL_CALLS: "tool_calls", FinishReason.CANCELLED: "stop", FinishReason.ERROR: "stop",
            None: "stop"}[r]


def _finish_anthropic(r: Optional[FinishReason]) -> str:
    return {FinishReason.STOP: "end_turn", FinishReason.STOP_SEQUENCE: "stop_sequence", FinishReason.LENGTH: "max_tokens",
            FinishReason.TOOL_CALLS: "tool_use", FinishReason.CANCELLED: "end_turn", FinishReason.ERROR: "end_turn",
            None: "end_turn"}[r]


def _usage_openai(u: Optional[Usage]) -> dict:
    u = u or Usage()
    return {"prompt_tokens": u.prompt_tokens, "completion_tokens": u.completion_tokens, "total_tokens": u.total_tokens,
            "prompt_tokens_details": {"cached_tokens": u.cached_tokens}}


def _timings(u: Optional[Usage]) -> dict:
    u = u or Usage()
    return {"queue_ms": round(u.queue_ms, 3), "prefill_ms": round(u.prefill_ms, 3), "decode_ms": round(u.decode_ms, 3),
            "cached_tokens": u.cached_tokens, "draft_tokens": u.draft_tokens, "accepted_tokens": u.accepted_tokens,
            "decode_tokens_per_second": round(u.completion_tokens / (u.decode_ms / 1000.0), 2) if u.decode_ms > 0 else None}


def _logprobs_openai(lps) -> Optional[dict]:
    if not lps:
        return None
    return {"content": [{"token": l.token, "logprob": l.logprob, "bytes": list(l.token.encode()),
                         "top_logprobs": [{"token": t.token, "logprob": t.logprob, "bytes": list(t.token.encode())}
                                          for t in l.top]} for l in lps]}


def _sse(obj) -> bytes:
    return b"data: " + json.dumps(obj, ensure_ascii=False).encode() + b"\n\n"


def _sse_event(name: str, obj) -> bytes:
    return f"event: {name}\n".encode() + b"data: " + json.dumps(obj, ensure_ascii=False).encode() + b"\n\n"


def create_app(engine: Engine, cfg: Optional[ServerConfig] = None) -> FastAPI:
    cfg = cfg or ServerConfig()
    app = FastAPI(title="legion-b200", version=__version__, docs_url=None, redoc_url=None)
    metrics = Metrics()
    logs = LogRing(2000)
    logging.getLogger("legion").addHandler(logs)
    app.state.engine, app.state.cfg, app.state.metrics, app.state.logs = engine, cfg, metrics, logs
    app.state.in_flight = 0
    started = time.time()

    def is_anthropic(path: str) -> bool:
        return path.startswith("/v1/messages")

    def err(path: str, status: int, message: str, kind: str = "invalid_request_error", param=None):
        if is_anthropic(path):
            amap = {401: "authentication_error", 404: "not_found_error", 413: "request_too_large", 429: "rate_limit_error",
                    529: "overloaded_error", 500: "api_error"}
            return _anthropic_error(status, message, amap.get(status, kind))
        omap = {401: "authentication_error", 404: "not_found_error", 429: "rate_limit_exceeded", 500: "server_error"}
        return _openai_error(status, message, omap.get(status, kind), param)

    @app.middleware("http")
    async def pipeline(request: Request, call_next):
        path = request.url.path
        rid = request.headers.get("x-request-id") or uuid.uuid4().hex
        request.state.request_id = rid
        t0 = time.perf_counter()
        if request.method == "OPTIONS" and cfg.cors:
            resp = PlainTextResponse("", status_code=204)
        elif cfg.api_keys and path not in ("/health", "/") and not path.startswith("/static"):
            key = request.headers.get("x-api-key")
            auth = request.headers.get("authorization", "")
            if not key and auth.lower().startswith("bearer "):
                key = auth[7:].strip()
            if key not in cfg.api_keys:
                resp = err(path, 401, "missing or invalid API key")
            else:
                request.state.share_key = key
                resp = None
        else:
            resp = None
        if resp is None:
            cl = request.headers.get("content-length")
            if cl and cl.isdigit() and int(cl) > cfg.max_request_mb * (1 << 20):
                resp = err(path, 413, f"request body exceeds {cfg.max_request_mb} MiB")
        if resp is None:
            app.state.in_flight += 1
            metrics.in_flight.set(app.state.in_flight)
            try:
                resp = await call_next(request)
            finally:
                app.state.in_flight -= 1
                metrics.in_flight.set(app.state.in_flight)
        resp.headers["x-request-id"] = rid
        if cfg.cors:
            resp.headers["access-control-allow-origin"] = "*"
            resp.headers["access-control-allow-headers"] = "*"
            resp.headers["access-control-allow-methods"] = "GET, POST, OPTIONS"
        metrics.http_requests.labels(path=path, method=request.method, status=str(resp.status_code)).inc()
        metrics.request_latency.labels(path=path).observe(time.perf_counter() - t0)
        return resp

    async def read_json(request: Request) -> dict:
        raw = await request.body()
        if len(raw) > cfg.max_request_mb * (1 << 20):
            raise ApiError(413, f"request body exceeds {cfg.max_request_mb} MiB")
        try:
            body = json.loads(raw or b"{}")
        except ValueError as e:
            raise ApiError(400, f"invalid JSON: {e}") from None
        if not isinstance(body, dict):
            raise ApiError(400, "request body must be a JSON object")
        return body

    def resolve_model(name: str) -> str:
        """Any name is accepted when one model is loaded; aliases map to the served id."""
        models = [m["id"] for m in engine.models()]
        name = cfg.model_aliases.get(name, name)
        if name in models or len(models) == 1:
            return models[0] if name not in models else name
        raise ApiError(404, f"model {name!r} is not served", kind="not_found_error", param="model")

    def submit(req: GenerateRequest, request: Request):
        req.request_id = request.state.request_id
        req.share_key = getattr(request.state, "share_key", None) if cfg.fair_share else None
        req.model = resolve_model(req.model)
        if req.response_format:
            try:
                engine.check_response_format(req.response_format)
            except ValueError as e:
                raise ApiError(400, f"response_format: {e}", param="response_format") from None
        try:
            return engine.generate(req)
        except EngineOverloaded as e:
            raise ApiError(529 if is_anthropic(request.url.path) else 429, str(e), kind="overloaded_error") from None
        except KvOverflow as e:
            raise ApiError(400, str(e), param="max_tokens") from None
        except ValueError as e:
            raise ApiError(400, str(e)) from None

    async def watch_disconnect(request: Request, stream):
        try:
            while True:
                if await request.is_disconnected():
                    stream.cancel()
                    return
                await asyncio.sleep(0.25)
        except asyncio.CancelledError:
            pass

    class Meter:
        """Per-request TTFT / ITL / token metrics."""

        def __init__(self):
            self.t0 = time.perf_counter()
            self.last = None

        def token(self):
            now = time.perf_counter()
            if self.last is None:
                metrics.ttft.observe(now - self.t0)
            else:
                metrics.itl.observe(now - self.last)
            self.last = now

        def done(self, usage: Optional[Usage]):
            if usage:
                metrics.prompt_tokens.inc(usage.prompt_tokens)
                metrics.completion_tokens.inc(usage.completion_tokens)

    @app.exception_handler(ApiError)
    async def api_error_handler(request: Request, e: ApiError):
        return err(request.url.path, e.status, e.message, e.kind, e.param)

    # ------------------------------------------------------------------ plain routes
    @app.get("/health")
    async def health():
        st = engine.stats()
        return {"status": "warming" if st.warming else "ok", "version": __version__, "git": os.environ.get("LEGION_GIT", ""),
                "uptime_s": round(time.time() - started, 1), "models": [m["id"] for m in engine.models()]}

    @app.get("/v1/models")
    @app.get("/models")
    async def models():
        return {"object": "list", "data": [dict(m, created=int(started)) for m in engine.models()]}

    @app.get("/v1/models/{model_id:path}")
    async def model(model_id: str, request: Request):
        for m in engine.models():
            if m["id"] == model_id or cfg.model_aliases.get(model_id) == m["id"]:
                return dict(m, created=int(started))
        return err(request.url.path, 404, f"model {model_id!r} is not served", "not_found_error")

    @app.get("/metrics")
    async def prom():
        metrics.update_engine(engine.stats())
        pctx = getattr(getattr(engine, "model", None), "pctx", None)
        if pctx is not None:
            metrics.update_parallel(pctx.stats)
        metrics.sample_gpus()
        return PlainTextResponse(metrics.render(), media_type="text/plain; version=0.0.4")

    def stats_snapshot() -> dict:
        st = engine.stats()
        return {"schema": 1, "time": time.time(), "uptime_s": round(time.time() - started, 1),
                "in_flight": app.state.in_flight, "engine": {
                    "running": st.running, "waiting": st.waiting, "waiting_by_priority": st.waiting_by_priority,
                    "kv_blocks_used": st.kv_blocks_used, "kv_blocks_total": st.kv_blocks_total,
                    "kv_preemptions": st.kv_preemptions, "prefix_cache_hit_tokens": st.prefix_cache_hit_tokens,
                    "prompt_tokens": st.prompt_tokens, "completion_tokens": st.completion_tokens, "steps": st.steps,
                    "step_ms": round(st.step_ms_ewma, 3), "warming": st.warming,
                    "spec": {"draft_tokens": st.spec_draft_tokens, "accepted_tokens": st.spec_accepted_tokens,
                             "acceptance_rate": round(st.spec_acceptance_rate, 4),
                             "mean_accepted_length": round(st.spec_mean_accepted_length, 3),
                             "verify_steps": st.spec_verify_steps}},
                "replicas": len(engine.replica_stats())}

    @app.get("/v1/stats")
    async def stats():
        return stats_snapshot()

    @app.get("/v1/stats/stream")
    async def stats_stream(request: Request):
        async def gen():
            while not await request.is_disconnected():
                yield _sse(stats_snapshot())
                await asyncio.sleep(1.0)
        return StreamingResponse(gen(), media_type="text/event-stream")

    @app.get("/v1/logs/stream")
    async def logs_stream(request: Request):
        async def gen():
            seen = 0
            while not await request.is_disconnected():
                lines, seen = logs.since(seen)
                for ln in lines:
                    yield _sse({"line": ln})
                await asyncio.sleep(0.5)
        return StreamingResponse(gen(), media_type="text/event-stream")

    @app.get("/")
    async def index():
        from .webui import INDEX_HTML
        return HTMLResponse(INDEX_HTML)

    # ------------------------------------------------------------------ OpenAI chat
    @app.post("/v1/chat/completions")
    async def chat_completions(request: Request):
        body = await read_json(request)
        req = convert.chat_request(body, cfg.sampling_defaults, cfg.default_max_tokens)
        stream = submit(req, request)
        cid = "chatcmpl-" + uuid.uuid4().hex[:24]
        created = int(time.time())
        model_id = req.model
        meter = Meter()
        include_usage = bool((body.get("stream_options") or {}).get("include_usage"))
        if body.get("stream"):
            async def gen() -> AsyncIterator[bytes]:
                watcher = asyncio.create_task(watch_disconnect(request, stream))
                n_calls = 0
                try:
                    first = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": model_id,
                             "choices": [{"index": 0, "delta": {"role": "assistant", "content": ""}, "finish_reason": None}]}
                    yield _sse(first)
                    async for ev in stream:
                        chunk = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": model_id}
                        if ev.kind == "text":
                            meter.token()
                            if not ev.text and not ev.logprobs:
                                continue
                            c = {"index": 0, "delta": {"content": ev.text}, "finish_reason": None}
                            lp = _logprobs_openai(ev.logprobs)
                            if lp:
                                c["logprobs"] = lp
                            chunk["choices"] = [c]
                            yield _sse(chunk)
                        elif ev.kind == "reasoning":
                            meter.token()
                            chunk["choices"] = [{"index": 0, "delta": {"reasoning_content": ev.text}, "finish_reason": None}]
                            yield _sse(chunk)
                        elif ev.kind == "tool_call":
                            tc = ev.tool_call
                            chunk["choices"] = [{"index": 0, "finish_reason": None, "delta": {"tool_calls": [
                                {"index": n_calls, "id": tc["id"], "type": "function",
                                 "function": {"name": tc["name"], "arguments": tc["arguments"]}}]}}]
                            n_calls += 1
                            yield _sse(chunk)
                        elif ev.kind == "finished":
                            meter.done(ev.usage)
                            chunk["choices"] = [{"index": 0, "delta": {}, "finish_reason": _finish_openai(ev.finish_reason)}]
                            chunk["timings"] = _timings(ev.usage)
                            yield _sse(chunk)
                            if include_usage:
                                yield _sse({"id": cid, "object": "chat.completion.chunk", "created": created,
                                            "model": model_id, "choices": [], "usage": _usage_openai(ev.usage)})
                        elif ev.kind == "error":
                            yield _sse({"error": {"message": ev.error, "type": "server_error"}})
                    yield b"data: [DONE]\n\n"
                finally:
                    watcher.cancel()
                    stream.cancel()
            return StreamingResponse(gen(), media_type="text/event-stream")
        comp = await collect(stream, request, meter)
        if comp.error:
            return err(request.url.path, comp.status or 500, comp.error, "server_error")
        msg: Dict[str, Any] = {"role": "assistant", "content": comp.text or (None if comp.tool_calls else "")}
        if comp.reasoning:
            msg["reasoning_content"] = comp.reasoning
        if comp.tool_calls:
            msg["tool_calls"] = [{"id": tc["id"], "type": "function",
                                  "function": {"name": tc["name"], "arguments": tc["arguments"]}} for tc in comp.tool_calls]
        choice = {"index": 0, "message": msg, "finish_reason": _finish_openai(comp.finish_reason)}
        lp = _logprobs_openai(comp.logprobs)
        if lp:
            choice["logprobs"] = lp
        return {"id": cid, "object": "chat.completion", "created": created, "model": model_id, "choices": [choice],
                "usage": _usage_openai(comp.usage), "timings": _timings(comp.usage)}

    async def collect(stream, request: Request, meter: Meter) -> Completion:
        watcher = asyncio.create_task(watch_disconnect(request, stream))
        comp = Completion()
        try:
            async for ev in stream:
                if ev.kind == "text":
                    meter.token()
                    comp.text += ev.text
                    comp.token_ids.extend(ev.token_ids)
                    comp.logprobs.extend(ev.logprobs)
                elif ev.kind == "reasoning":
                    meter.token()
                    comp.reasoning += ev.text
                elif ev.kind == "tool_call":
                    comp.tool_calls.append(ev.tool_call)
                elif ev.kind == "started":
                    comp.prompt_tokens = ev.prompt_tokens
                elif ev.kind == "finished":
                    comp.finish_reason, comp.usage = ev.finish_reason, ev.usage
                    meter.done(ev.usage)
                elif ev.kind == "error":
                    comp.error, comp.status = ev.error, ev.status
        finally:
            watcher.cancel()
        return comp

    # ------------------------------------------------------------------ OpenAI completions
    @app.post("/v1/completions")
    async def completions(request: Request):
        body = await read_json(request)
        req = convert.completion_request(body, cfg.sampling_defaults, 16)
        stream = submit(req, request)
        cid = "cmpl-" + uuid.uuid4().hex[:24]
        created = int(time.time())
        meter = Meter()
        if body.get("stream"):
            async def gen():
                watcher = asyncio.create_task(watch_disconnect(request, stream))
                try:
                    async for ev in stream:
                        base = {"id": cid, "object": "text_completion", "created": created, "model": req.model}
                        if ev.kind in ("text", "reasoning"):
                            meter.token()
                            base["choices"] = [{"index": 0, "text": ev.text, "finish_reason": None, "logprobs": None}]
                            yield _sse(base)
                        elif ev.kind == "finished":
                            meter.done(ev.usage)
                            base["choices"] = [{"index": 0, "text": "", "finish_reason": _finish_openai(ev.finish_reason),
                                                "logprobs": None}]
                            base["usage"] = _usage_openai(ev.usage)
                            yield _sse(base)
                        elif ev.kind == "error":
                            yield _sse({"error": {"message": ev.error, "type": "server_error"}})
                    yield b"data: [DONE]\n\n"
                finally:
                    watcher.cancel()
                    stream.cancel()
            return StreamingResponse(gen(), media_type="text/event-stream")
        comp = await collect(stream, request, meter)
        if comp.error:
            return err(request.url.path, comp.status or 500, comp.error, "server_error")
        text = ((req.prompt or "") if req.echo else "") + comp.reasoning + comp.text
        lp = None
        if comp.logprobs:
            lp = {"tokens": [l.token for l in comp.logprobs], "token_logprobs": [l.logprob for l in comp.logprobs],
                  "top_logprobs": [{t.token: t.logprob for t in l.top} for l in comp.logprobs]}
        return {"id": cid, "object": "text_completion", "created": created, "model": req.model,
                "choices": [{"index": 0, "text": text, "finish_reason": _finish_openai(comp.finish_reason), "logprobs": lp}],
                "usage": _usage_openai(comp.usage), "timings": _timings(comp.usage)}

    # ------------------------------------------------------------------ Anthropic messages
    @app.post("/v1/messages/count_tokens")
    async def count_tokens(request: Request):
        body = await read_json(request)
        b = dict(body)
        b.setdefault("max_tokens", 1)
        req = convert.anthropic_request(b, cfg.sampling_defaults)
        return {"input_tokens": engine.count_tokens(req)}

    @app.post("/v1/messages")
    async def messages(request: Request):
        body = await read_json(request)
        req = convert.anthropic_request(body, cfg.sampling_defaults)
        stream = submit(req, request)
        mid = "msg_" + uuid.uuid4().hex[:24]
        meter = Meter()
        if body.get("stream"):
            async def gen():
                watcher = asyncio.create_task(watch_disconnect(request, stream))
                idx = -1
                open_kind = None
                usage = Usage()
                try:
                    yield _sse_event("message_start", {"type": "message_start", "message": {
                        "id": mid, "type": "message", "role": "assistant", "model": req.model, "content": [],
                        "stop_reason": None, "stop_sequence": None, "usage": {"input_tokens": 0, "output_tokens": 0}}})
                    yield _sse_event("ping", {"type": "ping"})
                    reason = None

                    def close_block():
                        return _sse_event("content_block_stop", {"type": "content_block_stop", "index": idx})

                    async for ev in stream:
                        if ev.kind in ("text", "reasoning"):
                            meter.token()
                            kind = "thinking" if ev.kind == "reasoning" else "text"
                            if not ev.text:
                                continue
                            if open_kind != kind:
                                if open_kind is not None:
                                    yield close_block()
                                idx += 1
                                open_kind = kind
                                block = {"type": "thinking", "thinking": ""} if kind == "thinking" else {"type": "text", "text": ""}
                                yield _sse_event("content_block_start", {"type": "content_block_start", "index": idx,
                                                                         "content_block": block})
                            delta = {"type": "thinking_delta", "thinking": ev.text} if kind == "thinking" \
                                else {"type": "text_delta", "text": ev.text}
                            yield _sse_event("content_block_delta", {"type": "content_block_delta", "index": idx, "delta": delta})
                        elif ev.kind == "tool_call":
                            if open_kind is not None:
                                yield close_block()
                            idx += 1
                            open_kind = "tool_use"
                            tc = ev.tool_call
                            yield _sse_event("content_block_start", {"type": "content_block_start", "index": idx,
                                                                     "content_block": {"type": "tool_use", "id": tc["id"],
                                                                                       "name": tc["name"], "input": {}}})
                            yield _sse_event("content_block_delta", {"type": "content_block_delta", "index": idx,
                                                                     "delta": {"type": "input_json_delta",
                                                                               "partial_json": tc["arguments"]}})
                        elif ev.kind == "finished":
                            usage = ev.usage or usage
                            reason = ev.finish_reason
                            meter.done(ev.usage)
                        elif ev.kind == "error":
                            yield _sse_event("error", {"type": "error", "error": {"type": "api_error", "message": ev.error}})
                    if open_kind is not None:
                        yield close_block()
                    yield _sse_event("message_delta", {"type": "message_delta",
                                                       "delta": {"stop_reason": _finish_anthropic(reason), "stop_sequence": None},
                                                       "usage": {"input_tokens": usage.prompt_tokens,
                                                                 "output_tokens": usage.completion_tokens,
                                                                 "cache_read_input_tokens": usage.cached_tokens}})
                    yield _sse_event("message_stop", {"type": "message_stop"})
                finally:
                    watcher.cancel()
                    stream.cancel()
            return StreamingResponse(gen(), media_type="text/event-stream")
        comp = await collect(stream, request, meter)
        if comp.error:
            return err(request.url.path, comp.status or 500, comp.error, "api_error")
        content: List[dict] = []
        if comp.reasoning:
            content.append({"type": "thinking", "thinking": comp.reasoning})
        if comp.text or not comp.tool_calls:
            content.append({"type": "text", "text": comp.text})
        for tc in comp.tool_calls:
            try:
                inp = json.loads(tc["arguments"])
            except ValueError:
                inp = {"raw": tc["arguments"]}
            content.append({"type": "tool_use", "id": tc["id"], "name": tc["name"], "input": inp})
        u = comp.usage or Usage()
        return {"id": mid, "type": "message", "role": "assistant", "model": req.model, "content": content,
                "stop_reason": _finish_anthropic(comp.finish_reason), "stop_sequence": None,
                "usage": {"input_tokens": u.prompt_tokens, "output_tokens": u.completion_tokens,
                          "cache_read_input_tokens": u.cached_tokens, "cache_creation_input_tokens": 0}}

    # ------------------------------------------------------------------ OpenAI responses
    @app.post("/v1/responses")
    async def responses(request: Request):
        body = await read_json(request)
        req = convert.responses_request(body, cfg.sampling_defaults, cfg.default_max_tokens)
        stream = submit(req, request)
        rid = "resp_" + uuid.uuid4().hex[:24]
        created = int(time.time())
        meter = Meter()

        def envelope(status: str, output: list, usage: Optional[Usage]) -> dict:
            u = usage or Usage()
            return {"id": rid, "object": "response", "created_at": created, "status": status, "model": req.model,
                    "output": output, "usage": {"input_tokens": u.prompt_tokens, "output_tokens": u.completion_tokens,
                                                "total_tokens": u.total_tokens,
                                                "input_tokens_details": {"cached_tokens": u.cached_tokens}},
                    "store": False, "previous_response_id": None}

        def build_output(comp: Completion) -> list:
            out = []
            if comp.reasoning:
                out.append({"type": "reasoning", "id": "rs_" + uuid.uuid4().hex[:16],
                            "summary": [{"type": "summary_text", "text": comp.reasoning}]})
            if comp.text or not comp.tool_calls:
                out.append({"type": "message", "id": "msg_" + uuid.uuid4().hex[:16], "role": "assistant", "status": "completed",
                            "content": [{"type": "output_text", "text": comp.text, "annotations": []}]})
            for tc in comp.tool_calls:
                out.append({"type": "function_call", "id": "fc_" + uuid.uuid4().hex[:16], "call_id": tc["id"],
                            "name": tc["name"], "arguments": tc["arguments"], "status": "completed"})
            return out

        if body.get("stream"):
            async def gen():
                watcher = asyncio.create_task(watch_disconnect(request, stream))
                comp = Completion()
                seq = 0
                try:
                    yield _sse_event("response.created", {"type": "response.created", "sequence_number": seq,
                                                          "response": envelope("in_progress", [], None)})
                    async for ev in stream:
                        if ev.kind == "text":
                            meter.token()
                            comp.text += ev.text
                            if ev.text:
                                seq += 1
                                yield _sse_event("response.output_text.delta", {"type": "response.output_text.delta",
                                                                                "sequence_number": seq, "output_index": 0,
                                                                                "content_index": 0, "delta": ev.text})
                        elif ev.kind == "reasoning":
                            comp.reasoning += ev.text
                        elif ev.kind == "tool_call":
                            comp.tool_calls.append(ev.tool_call)
                        elif ev.kind == "finished":
                            comp.usage, comp.finish_reason = ev.usage, ev.finish_reason
                            meter.done(ev.usage)
                        elif ev.kind == "error":
                            comp.error = ev.error
                    seq += 1
                    status = "failed" if comp.error else ("incomplete" if comp.finish_reason == FinishReason.LENGTH else "completed")
                    yield _sse_event("response.completed", {"type": "response.completed", "sequence_number": seq,
                                                            "response": envelope(status, build_output(comp), comp.usage)})
                finally:
                    watcher.cancel()
                    stream.cancel()
            return StreamingResponse(gen(), media_type="text/event-stream")
        comp = await collect(stream, request, meter)
        if comp.error:
            return err(request.url.path, comp.status or 500, comp.error, "server_error")
        status = "incomplete" if comp.finish_reason == FinishReason.LENGTH else "completed"
        resp = envelope(status, build_output(comp), comp.usage)
        resp["output_text"] = comp.text
        return resp

    return app


def serve(engine: Engine, host: str = "127.0.0.1", port: int = 8090, cfg: Optional[ServerConfig] = None,
          tls_cert: Optional[str] = None, tls_key: Optional[str] = None, log_level: str = "info"):
    """Runs the server until interrupted; in-flight requests get ``shutdown_timeout_s`` to finish."""
    import uvicorn
    cfg = cfg or ServerConfig()
    app = create_app(engine, cfg)
    uv = uvicorn.Config(app, host=host, port=port, log_level=log_level, ssl_certfile=tls_cert, ssl_keyfile=tls_key,
                        timeout_graceful_shutdown=int(cfg.shutdown_timeout_s))
    server = uvicorn.Server(uv)
    try:
        server.run()
    finally:
        engine.shutdown()
