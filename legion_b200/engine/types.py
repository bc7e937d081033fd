"""Wire-neutral request / response types and the ``Engine`` interface.

The HTTP layer converts OpenAI / Anthropic requests into ``GenerateRequest`` and renders ``TokenEvent``s
back in the caller's API shape; engines (``LmEngine``, ``MockEngine``, ``ReplicaEngine``) implement
``Engine``. Mirrors ``src/engine/mod.rs:26-378`` of the reference (GenerateRequest :157-184, TokenEvent
:235-260, EngineStats :285-328, trait Engine :338-378).
"""
from __future__ import annotations

import asyncio
import queue
import threading
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, Iterator, List, Optional, Sequence, Union


class FinishReason(str, Enum):
    STOP = "stop"                  # end-of-sequence token
    STOP_SEQUENCE = "stop_sequence"
    LENGTH = "length"
    TOOL_CALLS = "tool_calls"
    CANCELLED = "cancelled"
    ERROR = "error"


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    seed: Optional[int] = None
    max_tokens: int = 4096
    min_tokens: int = 0
    stop: List[str] = field(default_factory=list)
    stop_token_ids: List[int] = field(default_factory=list)
    ignore_eos: bool = False
    logprobs: bool = False
    top_logprobs: int = 0
    logit_bias: Dict[int, float] = field(default_factory=dict)

    def validate(self, anthropic: bool = False):
        hi = 1.0 if anthropic else 2.0
        if not (0.0 <= self.temperature <= hi):
            raise ValueError(f"temperature must be between 0 and {hi:g}")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if not (0.0 <= self.min_p <= 1.0):
            raise ValueError("min_p must be between 0 and 1")
        for name in ("presence_penalty", "frequency_penalty"):
            if not (-2.0 <= getattr(self, name) <= 2.0):
                raise ValueError(f"{name} must be between -2 and 2")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be positive")
        if not (0 <= self.top_logprobs <= 20):
            raise ValueError("top_logprobs must be between 0 and 20")
        if self.min_tokens > self.max_tokens:
            raise ValueError("min_tokens must not exceed max_tokens")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def plain(self) -> bool:
        """No host-side logit edits needed: the device can pick the token."""
        return (self.presence_penalty == 0 and self.frequency_penalty == 0 and self.repetition_penalty == 1.0
                and not self.logit_bias and not self.logprobs and self.min_tokens == 0)


@dataclass
class ChatMessage:
    role: str
    content: Union[str, List[dict]] = ""
    tool_calls: Optional[List[dict]] = None
    tool_call_id: Optional[str] = None
    name: Optional[str] = None
    reasoning_content: Optional[str] = None


@dataclass
class GenerateRequest:
    model: str = ""
    messages: Optional[List[ChatMessage]] = None     # chat form (rendered through the chat template)
    prompt: Optional[str] = None                     # raw text completion
    prompt_tokens: Optional[List[int]] = None        # already tokenised
    sampling: SamplingParams = field(default_factory=SamplingParams)
    tools: Optional[List[dict]] = None
    tool_choice: Optional[Any] = None
    response_format: Optional[dict] = None           # {"type": "json_schema"|"json_object", ...}
    enable_thinking: Optional[bool] = None
    images: List[bytes] = field(default_factory=list)
    priority: int = 0
    share_key: Optional[str] = None                  # fair-share bucket
    request_id: str = ""
    add_generation_prompt: bool = True
    echo: bool = False


@dataclass
class Usage:
    prompt_tokens: int = 0
    completion_tokens: int = 0
    cached_tokens: int = 0
    queue_ms: float = 0.0
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    draft_tokens: int = 0
    accepted_tokens: int = 0

    @property
    def total_tokens(self) -> int:
        return self.prompt_tokens + self.completion_tokens


@dataclass
class TokenLogprob:
    token: str
    token_id: int
    logprob: float
    top: List["TokenLogprob"] = field(default_factory=list)


@dataclass
class TokenEvent:
    kind: str                                  # started | text | reasoning | tool_call | finished | error
    text: str = ""
    token_ids: List[int] = field(default_factory=list)
    logprobs: List[TokenLogprob] = field(default_factory=list)
    prompt_tokens: int = 0
    finish_reason: Optional[FinishReason] = None
    usage: Optional[Usage] = None
    tool_call: Optional[dict] = None           # {"id", "name", "arguments"}
    error: Optional[str] = None
    status: int = 500


class CancelToken:
    def __init__(self):
        self._ev = threading.Event()

    def cancel(self):
        self._ev.set()

    @property
    def cancelled(self) -> bool:
        return self._ev.is_set()


class TokenStream:
    """Events of one request. Iterable from a thread (``for ev in stream``) or from asyncio
    (``async for ev in stream``). The producer is the engine thread."""

    _END = object()

    def __init__(self, cancel: Optional[CancelToken] = None):
        self._q: "queue.Queue" = queue.Queue()
        self.cancel_token = cancel or CancelToken()
        self._done = False

    # producer side
    def put(self, ev: TokenEvent):
        self._q.put(ev)
        if ev.kind in ("finished", "error"):
            self._q.put(self._END)

    def cancel(self):
        self.cancel_token.cancel()

    # consumer side
    def get(self, timeout: Optional[float] = None):
        if self._done:
            return None
        try:
            ev = self._q.get(timeout=timeout)
        except queue.Empty:
            raise TimeoutError
        if ev is self._END:
            self._done = True
            return None
        return ev

    def __iter__(self) -> Iterator[TokenEvent]:
        while True:
            ev = self.get()
            if ev is None:
                return
            yield ev

    def __aiter__(self):
        return self

    async def __anext__(self) -> TokenEvent:
        loop = asyncio.get_running_loop()
        while True:
            try:
                ev = await loop.run_in_executor(None, self.get, 0.25)
            except TimeoutError:
                continue
            if ev is None:
                raise StopAsyncIteration
            return ev

    def collect(self) -> "Completion":
        """Blocks until the request ends and returns the assembled reply."""
        c = Completion()
        for ev in self:
            if ev.kind == "text":
                c.text += ev.text
                c.token_ids.extend(ev.token_ids)
                c.logprobs.extend(ev.logprobs)
            elif ev.kind == "reasoning":
                c.reasoning += ev.text
                c.token_ids.extend(ev.token_ids)
            elif ev.kind == "tool_call":
                c.tool_calls.append(ev.tool_call)
                c.token_ids.extend(ev.token_ids)
            elif ev.kind == "started":
                c.prompt_tokens = ev.prompt_tokens
            elif ev.kind == "finished":
                c.finish_reason, c.usage = ev.finish_reason, ev.usage
            elif ev.kind == "error":
                c.error, c.status = ev.error, ev.status
                c.finish_reason = FinishReason.ERROR
        return c


@dataclass
class Completion:
    text: str = ""
    reasoning: str = ""
    token_ids: List[int] = field(default_factory=list)
    logprobs: List[TokenLogprob] = field(default_factory=list)
    tool_calls: List[dict] = field(default_factory=list)
    prompt_tokens: int = 0
    finish_reason: Optional[FinishReason] = None
    usage: Optional[Usage] = None
    error: Optional[str] = None
    status: int = 200


@dataclass
class EngineStats:
    running: int = 0
    waiting: int = 0
    waiting_by_priority: Dict[int, int] = field(default_factory=dict)
    waiting_keys: int = 0
    kv_blocks_used: int = 0
    kv_blocks_total: int = 0
    kv_preemptions: int = 0
    kv_swap_out: int = 0               # preempted sequences whose KV / state went to the host tier
    kv_swap_in: int = 0                # ... and came back instead of being recomputed
    prefix_host_spilled: int = 0       # prefix-cache blocks whose contents went to the host tier when evicted
    prefix_host_restored: int = 0      # ... and were copied back for a later prompt with that prefix
    prefix_cache_hit_tokens: int = 0
    prefix_cache_lookup_tokens: int = 0
    prompt_tokens: int = 0
    completion_tokens: int = 0
    steps: int = 0
    spec_draft_tokens: int = 0
    spec_accepted_tokens: int = 0
    spec_verify_steps: int = 0
    spec_mean_k: float = 0.0
    model_bytes_step: int = 0
    masks_ahead: int = 0               # grammar masks computed by helper threads beside the forward pass
    step_ms_ewma: float = 0.0
    # host time per step by phase, accumulated ms (plan = drafts + row planning, build = batch tensors + H2D,
    # forward = launches (+ wait for logits), finish = sampling / verification / text / stream events)
    host_ms: dict = field(default_factory=lambda: {"plan": 0.0, "build": 0.0, "forward": 0.0, "finish": 0.0})
    warming: bool = False

    @property
    def spec_acceptance_rate(self) -> float:
        return self.spec_accepted_tokens / self.spec_draft_tokens if self.spec_draft_tokens else 0.0

    @property
    def spec_mean_accepted_length(self) -> float:
        return 1.0 + self.spec_accepted_tokens / self.spec_verify_steps if self.spec_verify_steps else 0.0


class EngineOverloaded(Exception):
    """Waiting queue full: rendered as 429 (OpenAI) / 529 (Anthropic)."""


class KvOverflow(ValueError):
    """Prompt + max_tokens can never fit the KV cache: rendered as HTTP 400."""


class Engine:
    """What the server needs from an engine."""

    def models(self) -> List[dict]:
        raise NotImplementedError

    def check_response_format(self, fmt: Optional[dict]) -> None:
        """Raises ValueError when the constraint cannot be compiled."""

    def generate(self, req: GenerateRequest) -> TokenStream:
        raise NotImplementedError

    def count_tokens(self, req: GenerateRequest) -> int:
        raise NotImplementedError

    def stats(self) -> EngineStats:
        return EngineStats()

    def replica_stats(self) -> List[EngineStats]:
        return [self.stats()]

    def set_warming(self, on: bool) -> None:
        pass

    def shutdown(self) -> None:
        pass


def now_ms() -> float:
    return time.monotonic() * 1000.0
