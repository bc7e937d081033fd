"""LmEngine: the continuous-batching scheduler around one model.

One engine thread owns the model, the KV pool, the recurrent-state pool and the prefix cache. Callers
tokenise on their own thread (``prepare``) and hand a job to the engine thread, which loops:

    drain arrivals -> cancellations -> admit (prefix match, state restore, KV reserve / on-demand)
    -> plan a step (all decoding sequences, 1 + drafts rows each; prompt chunks under the token budget,
       cut at prefix-cache save points) -> one forward -> sample / verify -> stream text -> commit
       recurrent state, save snapshots, insert finished prompts into the radix cache, draft for the
       next step.

Reference structure: ``src/engine/lm.rs`` (Worker::run :6709-6950, admit :6955, place :7059-7184, step
:8034-8164, plan_step :8170-8512, finish_step :8519-9158), admission modes ``docs/serving.md:662-693``,
preemption by recompute ``src/engine/lm/preempt.rs:1-25``.
"""
from __future__ import annotations

import queue
import threading
import time
import traceback
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..config import ModelConfig
from ..kv.blocks import BlockPool, BlockTable, OutOfBlocks
from ..kv.radix import RadixCache
from ..kv.saved_states import SavedStates
from ..loaders import chat_template as chat_tpl
from ..loaders.tokenizer import ByteTokenizer, Tokenizer
from ..models.decoder import Decoder, KvCache, StatePool, StepBatch
from ..parallel.context import ParallelCtx
from .queue import WaitQueue
from .sampling import Sampler, top_logprobs
from .text import ChatFormat, IncrementalDetokenizer, ReasoningSplitter, StopChecker, ToolCallParser
from .types import (CancelToken, Engine, EngineOverloaded, EngineStats, FinishReason, GenerateRequest, KvOverflow,
                    SamplingParams, TokenEvent, TokenLogprob, TokenStream, Usage, now_ms)


@dataclass
class EngineConfig:
    ctx_size: int = 8192
    max_seqs: int = 16
    max_batch_tokens: int = 1024
    prefill_chunk: int = 512
    block_size: int = 64
    kv_cache_tokens: Optional[int] = None       # None: max_seqs * ctx_size; -1: as many as fit the GPU (memory plan)
    gpu_memory_utilization: float = 0.92        # share of the device's memory the memory plan may fill
    kv_fit_check: bool = False                  # refuse to start when an explicit KV pool does not fit
    prefix_cache: bool = True
    prefix_cache_states: int = 8
    prefix_cache_interval: int = 0
    max_waiting: int = 1024
    default_max_tokens: int = 4096
    scheduling_policy: str = "fcfs"
    fair_share: bool = False
    kv_admission: str = "reserve"               # reserve | on-demand
    nvtx: bool = False                          # NVTX range around every eager step (for external profilers)
    kv_swap_gib: float = 0.0                    # host tier for preempted sequences (0 = recompute instead)
    kv_rings: bool = False                      # sliding-window layers keep only window + one step of K / V per sequence
    prefix_host_gib: float = 0.0                # host tier of the prefix cache: evicted blocks keep their contents
                                                # in pinned memory and come back on a later hit (0 = dropped)
    spec: str = "none"                          # none | ngram | suffix | mtp | mtp_ngram | draft | eagle3 | dflash
    spec_draft_model: Optional[str] = None      # eagle3: head checkpoint directory; draft: a model path (same vocabulary)
    spec_k: int = 4
    spec_max_batch: int = 8
    spec_ngram_min: int = 2
    spec_ngram_max: int = 4
    deterministic: bool = False
    device: str = "cpu"
    seed: int = 0
    cuda_graphs: bool = True
    model_name: str = "legion-b200"
    tool_format: str = "hermes"
    reasoning: bool = True
    itl_target_ms: float = 0.0
    even_chunks: bool = True           # cut a prompt into equal chunks instead of full chunks + a short tail
    spec_policy: str = "fixed"        # fixed | cost | adaptive: draft depth per step from measured acceptance / costs
    spec_p_min: float = 0.5           # adaptive: a sequence drafts as deep as its last draft keeps this acceptance
    ttft_target_ms: float = 0.0


class _Swapped:
    """A preempted sequence's cache contents in host memory."""
    __slots__ = ("n_tokens", "nbytes", "k", "v", "conv", "ssm")

    def __init__(self, n_tokens: int, nbytes: int):
        self.n_tokens, self.nbytes = n_tokens, nbytes
        self.k, self.v, self.conv, self.ssm = {}, {}, {}, {}


class Seq:
    __slots__ = ("req", "stream", "tokens", "n_prompt", "n_computed", "table", "slot", "sampler", "detok", "stop",
                 "reason", "tools", "phase", "arrival_ms", "admit_ms", "first_ms", "usage", "radix_handle", "drafts",
                 "save_points", "finished", "priority", "key", "n_out", "held_logprobs", "constraint", "resumed", "swapped",
                 "orig_prompt", "last_hidden", "draft_state", "owner", "mask_ahead", "media", "spec_state", "spec_cap")

    def __init__(self, req: GenerateRequest, stream: TokenStream, tokens: List[int]):
        self.req, self.stream = req, stream
        self.tokens = list(tokens)
        self.n_prompt = len(tokens)
        self.orig_prompt = len(tokens)
        self.n_computed = 0
        self.swapped = None               # _Swapped: KV blocks + recurrent state parked in host memory
        self.media = None                 # vision.SeqMedia: image rows, their spans and rotary positions
        self.spec_state = None            # spec.depth.AdaptiveState under the adaptive draft-depth policy
        self.spec_cap = 0                 # the cap this step's drafts were made under
        self.table = BlockTable()
        self.slot = -1
        self.owner = -1                   # data-parallel attention: the rank that runs this sequence's attention
        self.phase = "wait"
        self.arrival_ms = now_ms()
        self.admit_ms = 0.0
        self.first_ms = 0.0
        self.usage = Usage(prompt_tokens=len(tokens))
        self.radix_handle = None
        self.drafts: List[int] = []
        self.save_points: List[int] = []
        self.finished = False
        self.priority = req.priority
        self.key = req.share_key
        self.n_out = 0
        self.held_logprobs: List[TokenLogprob] = []
        self.constraint = None
        self.mask_ahead = None        # the next token's vocabulary mask, being computed beside the forward pass
        self.resumed = 0
        self.last_hidden = None
        self.draft_state = None
        self.sampler = None
        self.detok = None
        self.stop = None
        self.reason = None
        self.tools = None

    def key_tokens(self, n: Optional[int] = None) -> List[int]:
        """The tokens as the prefix cache and the saved states key them: image tokens stand as ids derived from
        their image's hash, so two images behind the same placeholder id never share a cache entry."""
        t = self.tokens if n is None else self.tokens[:n]
        return t if self.media is None else self.media.key_tokens(t)

    def rope_pos(self, p: int) -> int:
        return p if self.media is None else self.media.rope_position(p)


class LmEngine(Engine):
    def __init__(self, model: Decoder, tokenizer: Tokenizer, cfg: Optional[EngineConfig] = None, drafter=None,
                 start: bool = True):
        self.model = model
        self.mcfg: ModelConfig = model.cfg
        self.tok = tokenizer
        self.cfg = cfg or EngineConfig()
        c = self.cfg
        dev = model.device
        self.device = dev
        self.hybrid = bool(self.mcfg.recurrent_layers())
        # data-parallel attention: this rank runs attention only for the sequences it owns. A sequence that reuses a
        # cached prefix belongs to the rank that computed the prefix (the blocks' contents exist only there);
        # otherwise to the rank with the fewest sequences.
        self.dp_world = getattr(model.pctx, "dp_world", 1)
        self.dp_rank = getattr(model.pctx, "dp_rank", 0)
        self._block_owner: Dict[int, int] = {}
        if self.dp_world > 1:
            if c.spec != "none" or drafter is not None:
                raise ValueError("speculative decoding is not available with data-parallel attention")
            c.prefix_host_gib = 0.0
            if self.hybrid:
                c.prefix_cache = False        # recurrent snapshots are not owner-aware
        # sliding-window rings (the reference's ``KvRing``, ``src/model/core/state.rs:38``): a sliding-window layer never
        # reads keys older than its window, so it keeps a short ring of blocks per sequence slot (window + the longest
        # step + one block) instead of pages for the whole context; logical block j of such a layer is ring block
        # j mod ring length. The prefix cache shares blocks of the common pool only; the rings' contents travel with
        # the state snapshots (``StatePool.attach_rings``), so a prompt resumes from the cache only where a snapshot
        # exists, as for recurrent layers. Preempted sequences are recomputed.
        self.ring_len = 0
        if c.kv_rings and "swa" in self.mcfg.layer_kinds and self.mcfg.sliding_window > 0:
            if self.dp_world > 1 or getattr(model, "pipe", None) is not None:
                raise ValueError("sliding-window rings are not available with data-parallel attention or pipeline stages")
            step = max(c.prefill_chunk, c.spec_k + 1 if (c.spec != "none" or drafter is not None) else 1)
            self.ring_len = (self.mcfg.sliding_window + step + c.block_size - 1) // c.block_size + 1
            c.kv_swap_gib = 0.0
            c.prefix_host_gib = 0.0
        kv_tokens = c.kv_cache_tokens or c.max_seqs * c.ctx_size
        n_blocks = max(4, (kv_tokens + c.block_size - 1) // c.block_size)
        extra = self.mcfg.mtp_layers if c.spec in ("mtp", "mtp_ngram") else 0
        owns = model.pipe.owns if getattr(model, "pipe", None) is not None else None
        self.memory_plan = None
        if dev.type == "cuda":
            n_blocks = self._plan_memory(model, dev, extra, owns, n_blocks)
        self.pool = BlockPool(n_blocks, c.block_size)
        # models whose prompts resume from the prefix cache only at state snapshots: recurrent layers, ring storage
        self.snap_resume = self.hybrid or bool(self.ring_len)
        n_saved = c.prefix_cache_states if (self.snap_resume and c.prefix_cache) else 0
        self.kv = KvCache(self.mcfg, n_blocks, c.block_size, dev, model.dtype, kv_heads_local=model.n_kv_l,
                          extra_layers=extra, owns=owns, ring_blocks=self.ring_len * (c.max_seqs + n_saved + 1))
        self.states = (StatePool(self.mcfg, c.max_seqs + n_saved + 1, dev, tp=model.pctx.tp, owns=owns)
                       if self.snap_resume else None)
        if self.ring_len:
            self.states.attach_rings(self.kv, self.ring_len,
                                     [il for il, k in enumerate(self.mcfg.layer_kinds)
                                      if k == "swa" and (not self.mcfg.sandwich_norm or self.mcfg.owns_kv(il))])
        self._free_slots = list(range(c.max_seqs - 1, -1, -1))
        self._slo = {"decode_ms": 0.0, "ms_per_prompt_token": 0.0}
        self._swap_bytes = 0
        self.radix = RadixCache(self.pool) if c.prefix_cache else None
        # host tier of the prefix cache: prefix hash -> (K rows, V rows) of one block over all layers, LRU order
        self._host_prefix: "Dict[bytes, Tuple[torch.Tensor, Optional[torch.Tensor]]]" = {}
        self._host_prefix_bytes = 0
        self.saved = SavedStates(range(c.max_seqs, c.max_seqs + n_saved), c.block_size) if n_saved else None
        self.waiting = WaitQueue(c.scheduling_policy, c.fair_share, c.max_waiting)
        self.running: List[Seq] = []
        self._inbox: "queue.Queue" = queue.Queue()
        self._stats = EngineStats(kv_blocks_total=n_blocks)
        self._warming = False
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._fail: Optional[str] = None
        if ("kda" in self.mcfg.layer_kinds) and (drafter is not None or c.spec != "none"):
            raise ValueError("speculative decoding is not available for models with Kimi-delta-attention layers "
                             "(their verify steps have no state replay)")
        self._depth_model = None          # spec.depth.DepthModel under the adaptive draft-depth policy
        self._draft_ms_step = 0.0
        self.vision = None                # vision.VisionRuntime once a tower is attached (``attach_vision``)
        self.drafter = drafter
        if self.drafter is None and c.spec != "none":
            from ..spec import make_drafter
            self.drafter = make_drafter(c.spec, self, **self._drafter_args())
        # reasoning markers, tool-call notation and further end-of-turn tokens, read from the vocabulary
        self.chat_format = ChatFormat(self.tok, c.tool_format)
        self.eos_ids = tuple(dict.fromkeys(list(self.tok.eos_ids) + list(self.chat_format.stop_ids)))
        self._graphs = None
        self._mask_pool = None
        caches_ok = all(getattr(ec, "graph_safe", False) for ec in model.expert_cache.values())
        if dev.type == "cuda" and c.cuda_graphs and caches_ok and getattr(model, "pipe", None) is None \
                and self._mamba_graphable() and self._mla_graphable(model, c) and not self.ring_len:
            from .cuda_graphs import DecodeGraphs
            self._graphs = DecodeGraphs(self)
        self.step_hook: Optional[Callable] = None    # tests observe (batch description) per step
        self.channel = None                          # parallel.spmd.StepChannel when several ranks serve together
        self._by_id: Dict[str, Seq] = {}
        if start:
            self.start()

    def _plan_memory(self, model, dev, extra, owns, n_blocks: int) -> int:
        """Sizes the KV pool against what the device has free beside the resident weights (``kv_cache_tokens = -1``:
        as many blocks as fit, up to every sequence's whole context) or checks that the asked pool fits, and logs
        the plan. An explicit pool that does not fit raises here, before anything large is allocated."""
        import logging

        from . import memory_plan as mp
        c = self.cfg
        probe = KvCache(self.mcfg, 1, c.block_size, dev, model.dtype, kv_heads_local=model.n_kv_l, extra_layers=extra,
                        owns=owns)
        bpb = probe.bytes_per_block()
        bpb_ring = probe.bytes_per_block(swa_only=True) if self.ring_len else 0
        del probe
        snap = self.hybrid or bool(self.ring_len)
        n_saved = c.prefix_cache_states if (snap and c.prefix_cache) else 0
        # ring storage: the sliding-window layers cost a fixed ring per sequence slot, not a share of every block
        bpb -= bpb_ring
        state_bytes = bpb_ring * self.ring_len * (c.max_seqs + n_saved + 1)
        if self.hybrid:
            sp = StatePool(self.mcfg, 1, dev, tp=model.pctx.tp, owns=owns)
            state_bytes += sp.bytes_per_slot() * (c.max_seqs + n_saved + 1)
            del sp
        free, total = torch.cuda.mem_get_info(dev)
        m = self.mcfg
        ws = mp.workspace_reserve(m.hidden, m.vocab, c.max_batch_tokens, c.max_seqs, m.n_expert, m.top_k, m.expert_ff)
        auto = c.kv_cache_tokens is not None and c.kv_cache_tokens < 0
        asked = 0 if auto else n_blocks * c.block_size
        plan = mp.fit(total, free, torch.cuda.memory_allocated(dev), bpb, c.block_size, state_bytes, ws, c.max_seqs,
                      c.ctx_size, asked_tokens=asked, utilisation=c.gpu_memory_utilization)
        self.memory_plan = plan
        log = logging.getLogger("legion")
        for line in plan.lines():
            log.info(line)
        if auto:
            return plan.n_blocks
        if not plan.fits and c.kv_fit_check:
            raise ValueError("the KV pool does not fit this GPU: " + "; ".join(plan.lines()[1:]))
        return n_blocks

    def _drafter_args(self) -> dict:
        """``spec_draft_model``: the EAGLE-3 head checkpoint, or the draft model, the drafter is built from."""
        c = self.cfg
        if not c.spec_draft_model:
            return {}
        if c.spec == "eagle3":
            from ..spec.drafters import Eagle3Head
            return {"head": Eagle3Head.from_checkpoint(c.spec_draft_model, self.mcfg, self.device, self.model.dtype)}
        if c.spec == "draft":
            from ..loaders.model import load_model
            dcfg, dw, _, _ = load_model(c.spec_draft_model, str(self.device))
            return {"draft": Decoder(dcfg, dw, None, max_position=c.ctx_size + 8)}
        return {}

    def _mamba_graphable(self) -> bool:
        """Mamba-2 layers decode from CUDA graphs when their head shape runs on the scan kernel (the token loop that
        serves other shapes reads sequence bounds on the host)."""
        m = self.mcfg
        if "kda" in m.layer_kinds or m.hyper_streams > 1 or m.sandwich_norm or m.block_form:
            return False          # forward paths built from tensor operations (no captured decode step)
        if "mamba2" not in m.layer_kinds:
            return True
        from ..ops import sm100
        return sm100.mamba2_scan_ok(m.ssm_heads, m.ssm_head_dim, m.ssm_groups, m.ssm_state)

    # ------------------------------------------------------------------ Engine interface
    def models(self):
        return [{"id": self.cfg.model_name, "object": "model", "owned_by": "legion-b200",
                 "context_length": self.cfg.ctx_size}]

    def start(self):
        if self._thread is None:
            self._thread = threading.Thread(target=self._run, name="legion-engine", daemon=True)
            self._thread.start()

    def shutdown(self):
        self._stop.set()
        self._inbox.put(None)
        if self._thread is not None:
            self._thread.join(timeout=30)
            self._thread = None
        if self._mask_pool is not None:
            self._mask_pool.shutdown(wait=False)
            self._mask_pool = None
        self.release_graphs()

    def release_graphs(self):
        """Drops the captured decode graphs. Graphs that captured NCCL collectives must be gone before the
        process group is destroyed (tearing the communicator down under live graphs can block)."""
        if self._graphs is not None:
            self._graphs.release()

    def set_warming(self, on: bool):
        self._warming = on
        self._stats.warming = on

    def stats(self) -> EngineStats:
        s = self._stats
        s.running, s.waiting = len(self.running), len(self.waiting)
        s.waiting_by_priority = self.waiting.by_priority()
        s.waiting_keys = self.waiting.n_keys()
        s.kv_blocks_used = self.pool.used
        if self.radix is not None:
            s.prefix_cache_hit_tokens = self.radix.hit_tokens
            s.prefix_cache_lookup_tokens = self.radix.lookup_tokens
        return s

    def check_response_format(self, fmt):
        if fmt:
            from ..grammar import compile_response_format
            compile_response_format(fmt, self.tok)

    def tokenize_request(self, req: GenerateRequest) -> List[int]:
        if req.prompt_tokens is not None:
            return list(req.prompt_tokens)
        if req.messages is not None:
            tpl = self.tok.chat_template
            if not tpl:
                raise ValueError("model has no chat template")
            kwargs = {}
            if req.enable_thinking is not None:
                kwargs["enable_thinking"] = req.enable_thinking
            text = chat_tpl.render(tpl, req.messages, tools=req.tools, add_generation_prompt=req.add_generation_prompt,
                                   **kwargs)
            return self.tok.encode(text, add_special=True)
        return self.tok.encode(req.prompt or "", add_special=True)

    def attach_vision(self, runtime) -> None:
        """Gives the engine a vision tower (``vision.VisionRuntime``): requests may then carry images. The
        placeholder and marker token ids are looked up in this engine's vocabulary."""
        runtime.bind_tokenizer(self.tok)
        if runtime.tower.cfg.out_hidden != self.mcfg.hidden:
            raise ValueError(f"vision tower rows are {runtime.tower.cfg.out_hidden} wide, the model takes {self.mcfg.hidden}")
        self.vision = runtime

    def _media_inputs(self, b: StepBatch, rows, tok: List[int]) -> None:
        """Steps that touch image tokens: the token embedding with the image rows in place, the extra rows of the
        first layers, and per-token rotary rows when the model turns its frequencies with three position axes."""
        dev = self.device
        for s, _, _ in rows:
            if s.media is not None and s.media.rows is None:
                s.media.materialize(self.vision, dev, self.model.embed_dtype())     # the tower runs on this thread
        idx: List[int] = []          # rows of this step that are image tokens
        src: List[Tuple[object, int]] = []
        base = 0
        need_table = False
        for s, p0, n in rows:
            m = s.media
            if m is not None and s.phase != "decode" and p0 < m.n_prompt:
                hi = min(p0 + n, m.n_prompt)
                r = m.row_of_pos[p0:hi]
                hit = (r >= 0).nonzero().flatten().tolist()
                for j in hit:
                    idx.append(base + j)
                    src.append((m, int(r[j])))
                need_table = need_table or (m.pos3 is not None and bool(hit))
            base += n
        if idx:
            x = self.model.embed(b.token_ids)
            groups = {}
            for at, (m, r) in zip(idx, src):
                groups.setdefault(id(m), (m, [], []))
                groups[id(m)][1].append(at)
                groups[id(m)][2].append(r)
            n_deep = min(len(m.deepstack) for m, _, _ in groups.values())
            deep = [torch.zeros(len(idx), x.shape[1], dtype=x.dtype, device=dev) for _ in range(n_deep)]
            order = {at: i for i, at in enumerate(idx)}
            for m, ats, rs in groups.values():
                at_t = torch.tensor(ats, dtype=torch.int64, device=dev)
                r_t = torch.tensor(rs, dtype=torch.int64, device=m.rows.device)
                x[at_t] = m.rows[r_t].to(device=dev, dtype=x.dtype)
                where = torch.tensor([order[a] for a in ats], dtype=torch.int64, device=dev)
                for j in range(n_deep):
                    deep[j][where] = m.deepstack[j][r_t].to(device=dev, dtype=x.dtype)
            b.embeds = x
            if n_deep:
                b.deepstack_rows = torch.tensor(idx, dtype=torch.int64, device=dev)
                b.deepstack = deep
        if need_table:
            pos3 = torch.zeros(3, len(tok), dtype=torch.int64)
            base = 0
            for s, p0, n in rows:
                m = s.media
                if m is not None and m.pos3 is not None:
                    hi = max(p0, min(p0 + n, m.n_prompt))
                    if hi > p0:
                        pos3[:, base:base + hi - p0] = m.pos3[:, p0:hi]
                    if p0 + n > hi:
                        pos3[:, base + hi - p0:base + n] = torch.arange(hi, p0 + n) + m.rope_delta
                else:
                    pos3[:, base:base + n] = torch.arange(p0, p0 + n)
                base += n
            b.rope_table = self.model.mrope_table(pos3)
            b.rope_rows = torch.arange(len(tok), dtype=torch.int32, device=dev)

    def count_tokens(self, req: GenerateRequest) -> int:
        return len(self.tokenize_request(req))

    def prepare(self, req: GenerateRequest) -> Seq:
        """Caller-thread half of ``generate``: template, tokenise, validate, compile the grammar."""
        req.sampling.validate()
        tokens = self.tokenize_request(req)
        if not tokens:
            tokens = [self.tok.bos_id if self.tok.bos_id is not None else 0]
        c = self.cfg
        media = None
        if req.images:
            if self.vision is None:
                raise ValueError("this model has no vision tower: images cannot be used (--mmproj)")
            tokens, media = self.vision.attach(tokens, req.images, self.mcfg.hidden, self.mcfg.mrope_sections is not None)
        if len(tokens) + 1 > c.ctx_size:
            raise KvOverflow(f"prompt of {len(tokens)} tokens does not fit the context of {c.ctx_size}")
        sp = req.sampling
        sp.max_tokens = min(sp.max_tokens, c.ctx_size - len(tokens))
        need = self.pool.blocks_for(len(tokens) + (sp.max_tokens if c.kv_admission == "reserve" else 1))
        if need > self.pool.total:
            raise KvOverflow(f"request needs {need} KV blocks, the cache has {self.pool.total}")
        seq = Seq(req, TokenStream(CancelToken()), tokens)
        seq.media = media
        if req.response_format and req.response_format.get("type") not in (None, "text"):
            from ..grammar import compile_response_format
            seq.constraint = compile_response_format(req.response_format, self.tok)
        return seq

    def generate(self, req: GenerateRequest) -> TokenStream:
        if self._fail:
            raise RuntimeError(self._fail)
        if self.waiting.full():
            raise EngineOverloaded("waiting queue is full")
        seq = self.prepare(req)
        self._inbox.put(seq)
        return seq.stream

    # ------------------------------------------------------------------ engine thread
    def _run(self):
        try:
            while not self._stop.is_set():
                idle = not self.running and len(self.waiting) == 0
                if self.channel is not None:
                    self._sync_ranks(idle)
                else:
                    self._drain(block=idle)
                    if self._stop.is_set():
                        break
                    self._handle_cancels()
                if self._stop.is_set():
                    break
                self._admit()
                if self.running:
                    self.step()
        except BaseException as e:  # a failed step ends every request with an error event
            self._fail = f"engine failed: {e!r}"
            traceback.print_exc()
            self._fail_all(self._fail)

    def _drain(self, block: bool):
        try:
            item = self._inbox.get(timeout=0.2) if block else self._inbox.get_nowait()
        except queue.Empty:
            return
        while True:
            if item is None:
                return
            self.waiting.push(item, item.priority, item.key)
            try:
                item = self._inbox.get_nowait()
            except queue.Empty:
                return

    def _sync_ranks(self, idle: bool):
        """Several ranks, one scheduler each: rank 0 publishes the requests and cancellations it saw since the
        last step; every rank applies them at the same step boundary, so all ranks plan the same steps."""
        import pickle
        ch = self.channel
        msgs = None
        if ch.rank == 0:
            msgs = []
            try:
                item = self._inbox.get(timeout=0.2) if idle else self._inbox.get_nowait()
                while True:
                    if item is None:
                        msgs.append(("shutdown", None))
                        break
                    if not item.req.request_id:
                        item.req.request_id = f"r{id(item):x}"
                    self._by_id[item.req.request_id] = item
                    msgs.append(("req", pickle.dumps(item.req)))
                    item = self._inbox.get_nowait()
            except queue.Empty:
                pass
            for s in list(self.running) + self.waiting.items():
                if s.stream.cancel_token.cancelled and not s.finished:
                    msgs.append(("cancel", s.req.request_id))
        for kind, payload in ch.exchange(msgs):
            if kind == "shutdown":
                self._stop.set()
                return
            if kind == "req":
                req = pickle.loads(payload)
                seq = self._by_id.get(req.request_id) if ch.rank == 0 else None
                if seq is None:
                    seq = self.prepare(req)
                    self._by_id[req.request_id] = seq
                self.waiting.push(seq, seq.priority, seq.key)
            elif kind == "cancel":
                seq = self._by_id.get(payload)
                if seq is None or seq.finished:
                    continue
                if seq in self.running:
                    self._finish(seq, FinishReason.CANCELLED)
                else:
                    self.waiting.remove(lambda q: q is seq)
                    seq.finished = True
                    seq.stream.put(TokenEvent(kind="finished", finish_reason=FinishReason.CANCELLED, usage=seq.usage))

    def _fail_all(self, msg: str):
        for s in self.running + self.waiting.items():
            s.stream.put(TokenEvent(kind="error", error=msg, status=500))
        self.running.clear()

    def _handle_cancels(self):
        for s in list(self.running):
            if s.stream.cancel_token.cancelled:
                self._finish(s, FinishReason.CANCELLED)
        for s in self.waiting.remove(lambda q: q.stream.cancel_token.cancelled):
            s.stream.put(TokenEvent(kind="finished", finish_reason=FinishReason.CANCELLED, usage=s.usage))

    # ------------------------------------------------------------------ admission
    def _blocks_needed(self, seq: Seq, cached_blocks: int) -> int:
        total = seq.n_prompt + (seq.req.sampling.max_tokens - seq.n_out if self.cfg.kv_admission == "reserve"
                                else self.cfg.spec_k + 2)
        return max(0, self.pool.blocks_for(total) - cached_blocks)

    def _make_room(self, need: int, keep=None) -> bool:
        """Frees KV blocks until ``need`` are available: radix leaves first, then saved snapshots that pin a tail
        block (oldest first). ``keep`` is a snapshot the caller is about to resume from: it is never dropped."""
        if self.pool.free >= need:
            return True
        if self.radix is not None:
            spill = self._spill_prefix_block if (self.cfg.prefix_host_gib > 0 and not self.snap_resume) else None
            self.radix.evict(need - self.pool.free, spill)
        if self.pool.free < need and self.saved is not None:
            for s in sorted(self.saved.entries(), key=lambda e: e.tick):
                if s.tail_block is not None and s is not keep:
                    self.pool.decref(s.tail_block)
                    s.tail_block = None
                    self.saved.drop(s)
                    if self.pool.free >= need:
                        break
        return self.pool.free >= need

    # ------------------------------------------------------------------ prefix cache, host tier
    def _spill_prefix_block(self, prefix_tokens, block: int):
        """Eviction hook of the radix cache: the block's K/V rows of every layer go to pinned host memory under the
        hash of the prefix the block ends (``src/engine/lm/host_tier.rs`` keeps whole KV tails there; here the tier
        serves the prefix cache). Only blocks nobody else holds are kept: their contents are final."""
        from ..kv.saved_states import prefix_hashes
        if self.pool.refcount(block) != 1:
            return
        bs = self.cfg.block_size
        key = prefix_hashes(prefix_tokens, bs)[-1]
        if key in self._host_prefix:
            return
        layers = sorted(self.kv.k)
        k = torch.stack([self.kv.k[il][block] for il in layers]).cpu()
        shared = all(self.kv.v[il] is self.kv.k[il] for il in layers)
        v = None if shared else torch.stack([self.kv.v[il][block] for il in layers]).cpu()
        if self.device.type == "cuda":
            k = k.pin_memory()
            v = v.pin_memory() if v is not None else None
        nbytes = k.numel() * k.element_size() * (1 if v is None else 2)
        budget = self.cfg.prefix_host_gib * (1 << 30)
        while self._host_prefix and self._host_prefix_bytes + nbytes > budget:
            old_k, old_v = self._host_prefix.pop(next(iter(self._host_prefix)))
            self._host_prefix_bytes -= old_k.numel() * old_k.element_size() * (1 if old_v is None else 2)
        if nbytes > budget:
            return
        self._host_prefix[key] = (k, v)
        self._host_prefix_bytes += nbytes
        self._stats.prefix_host_spilled += 1

    def _restore_prefix_blocks(self, prompt, matched: int, limit: int, blocks: List[int]) -> int:
        """Continues a radix match from the host tier: while the next full block of the prompt is kept there, a
        device block is allocated, filled and inserted into the radix tree. Returns the number of blocks restored."""
        from ..kv.saved_states import prefix_hashes
        bs = self.cfg.block_size
        n_full = limit // bs
        if not self._host_prefix or matched // bs >= n_full:
            return 0
        hs = prefix_hashes(prompt[:n_full * bs], bs)
        layers = sorted(self.kv.k)
        new_blocks: List[int] = []
        i = matched // bs
        while i < n_full and hs[i] in self._host_prefix and self._make_room(1):
            if hs[i] not in self._host_prefix:          # making room spilled other blocks and pushed this one out
                break
            k, v = self._host_prefix.pop(hs[i])
            self._host_prefix[hs[i]] = (k, v)                       # most recently used last
            b = self.pool.alloc(1)[0]
            kd = k.to(self.device, non_blocking=True)
            vd = v.to(self.device, non_blocking=True) if v is not None else None
            for j, il in enumerate(layers):
                self.kv.k[il][b].copy_(kd[j])
                if vd is not None:
                    self.kv.v[il][b].copy_(vd[j])
            new_blocks.append(b)
            i += 1
        if new_blocks:
            self.radix.insert(prompt[:i * bs], list(blocks) + new_blocks)
            self.pool.release(new_blocks)                           # the tree holds them now
            self._stats.prefix_host_restored += len(new_blocks)
        return len(new_blocks)

    def _admit(self):
        c = self.cfg
        if c.deterministic and self.running:
            # admission waves: a batch is formed only when the engine is idle and runs to completion, so what a
            # request is batched with does not depend on when its neighbours arrived (``src/engine/lm/waves.rs``)
            return
        while len(self.waiting) and len(self.running) < c.max_seqs and self._free_slots:
            seq: Seq = self.waiting.peek()
            if not self._place(seq):
                break
            self.waiting.pop()

    def _place(self, seq: Seq) -> bool:
        """Prefix match + state restore + KV reservation. Returns False when the KV cache is too full."""
        bs = self.cfg.block_size
        prompt = seq.key_tokens()
        limit = len(prompt) - 1           # at least one prompt token is always recomputed
        blocks: List[int] = []
        matched = 0
        handle = None
        if self.radix is not None and limit >= bs and seq.swapped is None:
            blocks, matched, handle = self.radix.match_prefix(prompt, lock=True, max_tokens=limit)
            if self._host_prefix and not self.snap_resume and self._restore_prefix_blocks(prompt, matched, limit, blocks):
                self.radix.unlock(handle)
                blocks, matched, handle = self.radix.match_prefix(prompt, lock=True, max_tokens=limit)
        resume = matched
        saved = None
        tail_block = None
        if self.snap_resume:
            resume = 0
            if self.saved is not None and seq.swapped is None:
                cand = self.saved.find(prompt, limit)
                if cand is not None:
                    full = (cand.n_tokens // bs) * bs
                    if full <= matched and (cand.n_tokens == full or cand.tail_block is not None):
                        saved, resume = cand, cand.n_tokens
                        tail_block = cand.tail_block if cand.n_tokens != full else None
        use_blocks = blocks[:resume // bs]
        if handle is not None and len(use_blocks) < len(blocks):
            # matched blocks past the resume point are recomputed: do not keep them locked against eviction
            self.radix.unlock(handle)
            handle = None
            if use_blocks:
                blocks, matched, handle = self.radix.match_prefix(prompt, lock=True, max_tokens=len(use_blocks) * bs)
                use_blocks = blocks[:resume // bs]
        need = self._blocks_needed(seq, len(use_blocks) + (1 if tail_block is not None else 0))
        if not self._make_room(need, keep=saved):
            if handle is not None:
                self.radix.unlock(handle)
            if not self.running:
                # nothing will ever free memory for it
                self.waiting.remove(lambda q: q is seq)
                seq.stream.put(TokenEvent(kind="error", error="request does not fit the KV cache", status=400))
            return False
        seq.table = BlockTable.from_shared(self.pool, use_blocks, resume)
        if tail_block is not None:
            # the tail save is taken over by this sequence: its block moves into the table
            self.pool.incref(tail_block)
            seq.table.blocks.append(tail_block)
            self.pool.decref(tail_block)          # the snapshot's own reference
            saved.tail_block = None
        try:
            total = seq.n_prompt + (seq.req.sampling.max_tokens - seq.n_out if self.cfg.kv_admission == "reserve" else 1)
            seq.table.ensure(self.pool, total)
        except OutOfBlocks:
            seq.table.free(self.pool)
            if handle is not None:
                self.radix.unlock(handle)
            return False
        seq.radix_handle = handle
        seq.slot = self._free_slots.pop()
        if self.dp_world > 1 and not (seq.swapped is not None and seq.owner >= 0):
            if use_blocks:
                seq.owner = self._block_owner.get(use_blocks[0], 0)
            else:
                load = [sum(1 for r in self.running if r.owner == o) for o in range(self.dp_world)]
                seq.owner = load.index(min(load))
        if self.states is not None:
            if saved is not None:
                self.states.copy(saved.slot, seq.slot)
                if saved.kind == "tail":
                    self.saved.drop(saved)
            else:
                self.states.clear(seq.slot)
        if seq.swapped is not None:
            resume = self._swap_in(seq)          # KV blocks and recurrent state come back from the host tier
            seq.table.n_tokens = resume
        seq.n_computed = resume
        seq.resumed = resume
        seq.usage.cached_tokens = resume
        seq.phase = "prefill"
        seq.admit_ms = now_ms()
        seq.usage.queue_ms = seq.admit_ms - seq.arrival_ms
        if self.saved is not None:
            seq.save_points = self.saved.save_points(seq.n_prompt, resume, self.cfg.prefix_cache_interval)
        sp = seq.req.sampling
        if seq.sampler is None:     # a preempted sequence keeps its sampler and text state
            seq.sampler = Sampler(sp, seq.tokens, fallback_seed=self.cfg.seed)
            seq.detok = IncrementalDetokenizer(lambda ids: self.tok.decode(ids, skip_special=True))
            seq.stop = StopChecker(sp.stop)
            seq.reason = self.chat_format.splitter(self._prompt_tail(seq)) if self.cfg.reasoning else None
            seq.tools = ToolCallParser(self.chat_format.tool_format) if seq.req.tools else None
        if seq.n_out == 0:
            seq.stream.put(TokenEvent(kind="started", prompt_tokens=seq.orig_prompt))
        self.running.append(seq)
        self._stats.prompt_tokens += seq.n_prompt - resume
        return True

    def _prompt_tail(self, seq: Seq) -> str:
        """The end of the prompt as text (markers rendered): tells whether the template left a reasoning span open."""
        if isinstance(seq.req.prompt, str) and seq.req.prompt:
            return seq.req.prompt[-256:]
        try:
            return self.tok.decode(list(seq.tokens[max(0, seq.orig_prompt - 48):seq.orig_prompt]), skip_special=False)
        except Exception:
            return ""

    # ------------------------------------------------------------------ preemption (on-demand admission)
    def _preempt_one(self, protect: Seq) -> bool:
        """Frees the cheapest running sequence (lowest priority, fewest computed tokens, latest arrival);
        it is re-queued and recomputed later, its stream stays open."""
        cands = [s for s in self.running if s is not protect]
        if not cands:
            return False
        victim = min(cands, key=lambda s: (s.priority, s.n_computed, -s.arrival_ms))
        self._swap_out(victim)
        self._release(victim)
        self.running.remove(victim)
        victim.n_prompt = len(victim.tokens)
        victim.n_computed = 0
        victim.phase = "wait"
        victim.drafts = []
        self.waiting.requeue(victim, victim.priority, victim.key)
        self._stats.kv_preemptions += 1
        return True

    # ------------------------------------------------------------------ host tier for preempted sequences
    def _swap_out(self, s: Seq):
        """Parks the computed KV blocks (and the recurrent state) of a sequence about to be preempted in pinned
        host memory when the ``kv_swap_gib`` budget allows, so that re-admission copies them back instead of
        recomputing the prefix (the reference's ``KvTier``, ``src/model/core/kv_pool.rs``)."""
        c = self.cfg
        n = min(s.n_computed, len(s.tokens) - 1)
        if c.kv_swap_gib <= 0 or n < c.block_size or self.drafter is not None:
            return
        nb = self.pool.blocks_for(n)
        nbytes = nb * self.kv.bytes_per_block() + (self.states.bytes_per_slot() if self.states is not None else 0)
        if self._swap_bytes + nbytes > c.kv_swap_gib * (1 << 30):
            return
        idx = torch.tensor(s.table.blocks[:nb], dtype=torch.long, device=self.device)
        pin = self.device.type == "cuda"

        def park(t):
            h = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=pin)
            h.copy_(t, non_blocking=pin)
            return h
        sw = _Swapped(n, nbytes)
        for il, k in self.kv.k.items():
            sw.k[il] = park(k.index_select(0, idx))
            if self.kv.v[il] is not k:
                sw.v[il] = park(self.kv.v[il].index_select(0, idx))
        if self.states is not None and s.slot >= 0:
            sw.conv = {il: park(t[s.slot]) for il, t in self.states.conv.items()}
            sw.ssm = {il: park(t[s.slot]) for il, t in self.states.ssm.items()}
        if pin:
            torch.cuda.current_stream(self.device).synchronize()
        s.swapped = sw
        self._swap_bytes += nbytes
        self._stats.kv_swap_out += 1

    def _swap_in(self, s: Seq):
        """Copies a parked sequence back into its freshly reserved blocks / state slot. Returns the resumed length."""
        sw, s.swapped = s.swapped, None
        self._swap_bytes -= sw.nbytes
        nb = self.pool.blocks_for(sw.n_tokens)
        idx = torch.tensor(s.table.blocks[:nb], dtype=torch.long, device=self.device)
        for il, k in self.kv.k.items():
            k.index_copy_(0, idx, sw.k[il].to(self.device, non_blocking=True))
            if il in sw.v:
                self.kv.v[il].index_copy_(0, idx, sw.v[il].to(self.device, non_blocking=True))
        if self.states is not None:
            for il, t in sw.conv.items():
                self.states.conv[il][s.slot].copy_(t, non_blocking=True)
            for il, t in sw.ssm.items():
                self.states.ssm[il][s.slot].copy_(t, non_blocking=True)
        self._stats.kv_swap_in += 1
        return sw.n_tokens

    def _grow(self, seq: Seq, n_tokens: int) -> bool:
        while True:
            try:
                seq.table.ensure(self.pool, n_tokens)
                return True
            except OutOfBlocks:
                need = self.pool.blocks_for(n_tokens) - len(seq.table.blocks)
                if self._make_room(need):
                    continue
                if not self._preempt_one(seq):
                    return False

    # ------------------------------------------------------------------ one step
    # ------------------------------------------------------------------ step-time model (SLO budget, spec depth)
    def _observe_step(self, n_decode_rows: int, n_prompt_tokens: int, ms: float):
        """Two-parameter model of the step time: base (a decode-only step) + cost per prompt token, both EWMAs
        of what was measured (the reference's ``slo.rs`` fits the same shape from its step log)."""
        m = self._slo
        if n_prompt_tokens == 0:
            m["decode_ms"] = ms if m["decode_ms"] == 0 else 0.8 * m["decode_ms"] + 0.2 * ms
        elif n_prompt_tokens >= 32:
            per = max(0.0, ms - m["decode_ms"] * (1 if n_decode_rows else 0)) / n_prompt_tokens
            m["ms_per_prompt_token"] = per if m["ms_per_prompt_token"] == 0 else 0.8 * m["ms_per_prompt_token"] + 0.2 * per

    def slo_budget(self, n_decoding: int, first_chunk: bool) -> int:
        """Prompt tokens a step may carry so that decoding sequences keep ``itl_target_ms`` between tokens (or, with
        nothing decoding, so that a first chunk meets ``ttft_target_ms``). 0 = no limit known yet."""
        c, m = self.cfg, self._slo
        per = m["ms_per_prompt_token"]
        if per <= 0:
            return 0
        if n_decoding and c.itl_target_ms > 0:
            return max(16, int((c.itl_target_ms - m["decode_ms"]) / per))
        if first_chunk and c.ttft_target_ms > 0:
            return max(16, int(c.ttft_target_ms / per))
        return 0

    def _chunk_len(self, remaining: int, cap: int) -> int:
        """Length of the next prompt chunk: at most ``cap``; with even chunks the prompt's remainder is cut into
        equal parts (no short tail step, ``src/engine/lm/even.rs``)."""
        if remaining <= cap or not self.cfg.even_chunks:
            return min(remaining, cap)
        parts = -(-remaining // cap)
        return -(-remaining // parts)

    def _spec_depth(self, n_decode: int) -> int:
        """Draft depth for this step. ``cost`` policy: expected tokens per step with depth k is
        sum_{i<=k} p^i for acceptance rate p; a verify step of k extra rows per sequence costs about
        (1 + k * n_decode * row_cost) decode steps, so pick the k with the best tokens / cost ratio."""
        c = self.cfg
        if c.spec_policy not in ("cost", "adaptive"):
            return c.spec_k
        if c.spec_policy == "adaptive":
            return c.spec_k            # per-sequence caps and the measured-cost model decide in ``_adaptive_caps``
        st = self._stats
        drafted = max(1, st.spec_draft_tokens)
        p = min(0.98, max(0.05, st.spec_accepted_tokens / drafted)) if drafted > 32 else 0.6
        row_cost = 0.02                      # relative cost of one more verify row next to a decode step
        best_k, best = 0, 1.0
        for k in range(1, c.spec_k + 1):
            tokens = sum(p ** i for i in range(0, k + 1))
            cost = 1.0 + k * n_decode * row_cost
            if tokens / cost > best:
                best_k, best = k, tokens / cost
        return best_k

    def _adaptive_caps(self, decode) -> Dict[int, int]:
        """Adaptive policy (``spec/depth.py``): one depth for the step from the measured verify / draft costs and the
        sequences' expected gains, then per sequence the deepest draft whose last token keeps ``spec_p_min``
        acceptance; a sequence capped at 0 drafts one probing token every eighth step."""
        from ..spec.depth import AdaptiveState, DepthModel
        c = self.cfg
        if self._depth_model is None:
            self._depth_model = DepthModel(c.spec_k)
        cand = [s for s in decode if s.constraint is None]
        for s in cand:
            if s.spec_state is None:
                s.spec_state = AdaptiveState()
        step_k = self._depth_model.choose([s.spec_state for s in cand], len(cand)) if cand else 0
        caps = {}
        for s in cand:
            k = min(step_k, s.spec_state.cap(c.spec_p_min, c.spec_k))
            if k == 0 and s.spec_state.note_idle():
                k = 1
            caps[id(s)] = k
        return caps

    def step(self):
        t0 = time.perf_counter()
        c = self.cfg
        decode = [s for s in self.running if s.phase == "decode"]
        prefill = [s for s in self.running if s.phase == "prefill"]
        # drafts for this step (model-free drafters propose now; model drafters proposed after the last step)
        use_spec = self.drafter is not None and 0 < len(decode) <= c.spec_max_batch
        depth = self._spec_depth(len(decode)) if use_spec else 0
        caps = self._adaptive_caps(decode) if (use_spec and c.spec_policy == "adaptive") else None
        self._draft_ms_step = 0.0
        for s in decode:
            if caps is not None:
                depth = caps.get(id(s), 0)
            s.spec_cap = depth if use_spec else 0
            if not use_spec or s.constraint is not None or depth == 0:
                s.drafts = []
            elif self.drafter.model_free:
                s.drafts = self.drafter.propose(s, depth)
            else:
                s.drafts = s.drafts[:depth]
            room = s.req.sampling.max_tokens - s.n_out - 1
            s.drafts = s.drafts[:max(0, min(room, c.ctx_size - len(s.tokens) - 1))]
        rows: List[Tuple[Seq, int, int]] = []   # (seq, first position, n tokens)
        for s in list(decode):
            n = 1 + len(s.drafts)
            if c.kv_admission != "reserve" and not self._grow(s, len(s.tokens) + n):
                self._finish(s, FinishReason.LENGTH)
                continue
            if s not in self.running:
                continue
            rows.append((s, len(s.tokens) - 1, n))
        # token budget of the step: one for the whole step, or (data-parallel attention) one per owning rank, since
        # every rank runs only its own rows
        W = self.dp_world
        budgets = [c.max_batch_tokens - sum(r[2] for r in rows if W == 1 or r[0].owner == o) for o in range(W)]
        slo = self.slo_budget(len(rows), first_chunk=bool(prefill) and prefill[0].n_computed == 0)
        if slo:
            budgets = [min(b, slo) for b in budgets]
        for s in prefill:
            if s not in self.running:
                continue
            o = s.owner if W > 1 else 0
            budget = budgets[o]
            if budget <= 0:
                if W > 1:
                    continue
                break
            take = min(self._chunk_len(s.n_prompt - s.n_computed, c.prefill_chunk), budget)
            for sp in s.save_points:            # end the chunk at the next snapshot position
                if s.n_computed < sp < s.n_computed + take:
                    take = sp - s.n_computed
                    break
            if c.kv_admission != "reserve" and not self._grow(s, s.n_computed + take + 1):
                continue
            if s not in self.running:
                continue
            rows.append((s, s.n_computed, take))
            budgets[o] -= take
        rows = [r for r in rows if r[0] in self.running]
        if not rows:
            return
        self._stats.host_ms["plan"] += (time.perf_counter() - t0) * 1e3
        verify_rows = [r for r in rows if r[0].phase == "decode" and r[2] > 1]
        if self.hybrid and verify_rows:
            # speculative rows must not advance recurrent state: they run as their own pass with replay
            self._forward_and_finish(verify_rows, verify=True)
            rest = [r for r in rows if r not in verify_rows]
            if rest:
                self._forward_and_finish(rest, verify=False)
        else:
            self._forward_and_finish(rows, verify=False)
        dt = (time.perf_counter() - t0) * 1000
        if self._depth_model is not None and all(r[0].phase == "decode" or r[2] == 1 for r in rows):
            # a step of decode / verify rows only: its time (without the drafter's own passes) is V(rows)
            self._depth_model.observe_verify(sum(r[2] for r in rows), max(0.0, dt - self._draft_ms_step))
        self._observe_step(sum(1 for r in rows if r[0].phase == "decode" or r[2] == 1),
                           sum(r[2] for r in rows if r[2] > 1 and r not in verify_rows), dt)
        st = self._stats
        st.steps += 1
        st.step_ms_ewma = dt if st.step_ms_ewma == 0 else 0.8 * st.step_ms_ewma + 0.2 * dt

    def _mla_graphable(self, model, c) -> bool:
        """Latent-attention layers replay in a CUDA graph only through the tensor-core kernel (the fallback form
        reads lengths on the host)."""
        if "mla" not in self.mcfg.layer_kinds:
            return True
        from ..ops import sm100
        return sm100.mla_supported(model.n_head_l, self.mcfg.kv_lora, self.mcfg.qk_rope_dim, c.block_size)

    def build_batch(self, rows: Sequence[Tuple[Seq, int, int]], write_state: bool = True) -> StepBatch:
        dev = self.device
        tok: List[int] = []
        pos: List[int] = []
        slots: List[int] = []
        cu = [0]
        ctx: List[int] = []
        logit_rows: List[int] = []
        width = 1
        for s, p0, n in rows:
            if s.phase == "decode":
                toks = [s.tokens[-1]] + s.drafts[:n - 1]
            else:
                toks = s.tokens[p0:p0 + n]
            tok.extend(toks)
            if s.media is None:
                pos.extend(range(p0, p0 + n))
            else:
                pos.extend(s.rope_pos(p) for p in range(p0, p0 + n))
            slots.extend(s.table.slots(self.pool, p0, n))
            base = cu[-1]
            cu.append(base + n)
            ctx.append(p0 + n)
            width = max(width, self.pool.blocks_for(p0 + n))
            if s.phase == "decode":
                logit_rows.extend(range(base, base + n))
            elif p0 + n == s.n_prompt:
                logit_rows.append(base + n - 1)
        bt = torch.zeros(len(rows), width, dtype=torch.int32)
        for i, (s, p0, n) in enumerate(rows):
            nb = self.pool.blocks_for(p0 + n)
            bt[i, :nb] = torch.tensor(s.table.blocks[:nb], dtype=torch.int32)
        i32 = dict(dtype=torch.int32, device=dev)
        b = StepBatch(
            token_ids=torch.tensor(tok, **i32), positions=torch.tensor(pos, **i32), cu_q=torch.tensor(cu, **i32),
            ctx_lens=torch.tensor(ctx, **i32), block_table=bt.to(dev),
            slots=torch.tensor(slots, dtype=torch.int64, device=dev),
            state_slots=torch.tensor([s.slot for s, _, _ in rows], **i32),
            logit_rows=torch.tensor(logit_rows, dtype=torch.int64, device=dev),
            max_q_len=max(n for _, _, n in rows), max_ctx=max(ctx), write_state=write_state, cu_q_host=cu)
        if any(s.media is not None and s.phase != "decode" for s, _, _ in rows):
            self._media_inputs(b, rows, tok)
        if self.ring_len:
            self._ring_inputs(b, [(s, p0, n) for s, p0, n in rows], width)
        return b

    def _ring_inputs(self, b: StepBatch, rows, width: int) -> None:
        """KV cells and block table of the sliding-window layers: sequence slot s owns ring blocks
        [s * ring_len, (s + 1) * ring_len); position p lives in ring block (p // page) mod ring_len."""
        bs, L = self.cfg.block_size, self.ring_len
        cells: List[int] = []
        table = torch.zeros(len(rows), width, dtype=torch.int32)
        ring_of = torch.arange(width, dtype=torch.int32) % L
        for i, (s, p0, n) in enumerate(rows):
            base = s.slot * L
            cells.extend((base + (p // bs) % L) * bs + p % bs for p in range(p0, p0 + n))
            table[i] = base + ring_of
        b.slots_ring = torch.tensor(cells, dtype=torch.int64, device=self.device)
        b.block_table_ring = table.to(self.device)

    def build_batch_explicit(self, items, all_logits: bool = False) -> StepBatch:
        """items = [(seq, first position, token list)]: a batch over the sequences' own block tables with
        explicit tokens (drafters fill their KV and chain drafts with it). Logits: last row of each item."""
        dev = self.device
        tok, pos, slots, cu, ctx, lrows = [], [], [], [0], [], []
        width = 1
        for s, p0, toks in items:
            n = len(toks)
            tok.extend(toks)
            pos.extend(range(p0, p0 + n) if s.media is None else (s.rope_pos(p) for p in range(p0, p0 + n)))
            slots.extend(s.table.slots(self.pool, p0, n))
            cu.append(cu[-1] + n)
            ctx.append(p0 + n)
            width = max(width, self.pool.blocks_for(p0 + n))
            lrows.extend(range(cu[-2], cu[-1]) if all_logits else [cu[-1] - 1])
        bt = torch.zeros(len(items), width, dtype=torch.int32)
        for i, (s, p0, toks) in enumerate(items):
            nb = self.pool.blocks_for(p0 + len(toks))
            bt[i, :nb] = torch.tensor(s.table.blocks[:nb], dtype=torch.int32)
        i32 = dict(dtype=torch.int32, device=dev)
        b = StepBatch(token_ids=torch.tensor(tok, **i32), positions=torch.tensor(pos, **i32),
                      cu_q=torch.tensor(cu, **i32), ctx_lens=torch.tensor(ctx, **i32), block_table=bt.to(dev),
                      slots=torch.tensor(slots, dtype=torch.int64, device=dev),
                      state_slots=torch.tensor([s.slot for s, _, _ in items], **i32),
                      logit_rows=torch.tensor(lrows, dtype=torch.int64, device=dev),
                      max_q_len=max(len(t) for _, _, t in items), max_ctx=max(ctx), cu_q_host=cu)
        if self.ring_len:
            self._ring_inputs(b, [(s, p0, len(toks)) for s, p0, toks in items], width)
        return b

    def _own_blocks(self, s: Seq):
        """Data-parallel attention: blocks that enter the prefix cache remember which rank holds their contents."""
        if self.dp_world > 1:
            for b in s.table.blocks:
                self._block_owner[b] = s.owner

    def _dp_forward_and_finish(self, rows, verify: bool):
        """One step under data-parallel attention. Every rank plans the same global rows; this rank runs the model
        on the rows it owns (a padding row when it owns none, so that it still meets the others in every MoE
        layer's exchange), then the logit rows of all ranks are gathered into the global order and every rank
        samples all of them alike."""
        import torch.distributed as dist
        W, R = self.dp_world, self.dp_rank
        own = [r for r in rows if r[0].owner == R]
        if self._graphs is not None and all(
                s.phase == "decode" and n == 1 and s.req.sampling.greedy and s.req.sampling.plain and s.constraint is None
                for s, _, n in rows):
            # decode step from the graphs: every rank replays the bucket of the fullest rank, the picked tokens of
            # all ranks are gathered (one small collective) and mapped back to the global row order
            per_owner, where = [0] * W, []
            for s, _, _ in rows:
                where.append((s.owner, per_owner[s.owner]))
                per_owner[s.owner] += 1
            Bg = self._graphs.bucket(max(per_owner))
            if Bg is not None:
                picks, _ = self._graphs.run(own, B=Bg, gather=(self.model.pctx.dp_group, W))
                self._finish_rows(rows, None, None, None, verify, picked=[picks[o * Bg + off] for o, off in where])
                return
        if own:
            b = self.build_batch(own, write_state=not verify)
        else:
            i32 = dict(dtype=torch.int32, device=self.device)
            pad_slot = self.cfg.max_seqs + (self.cfg.prefix_cache_states if self.saved is not None else 0)
            b = StepBatch(token_ids=torch.zeros(1, **i32), positions=torch.zeros(1, **i32),
                          cu_q=torch.tensor([0, 1], **i32), ctx_lens=torch.ones(1, **i32),
                          block_table=torch.zeros(1, 1, **i32),
                          slots=torch.full((1,), -1, dtype=torch.int64, device=self.device),
                          state_slots=torch.full((1,), pad_slot, **i32),
                          logit_rows=torch.zeros(1, dtype=torch.int64, device=self.device), max_q_len=1, max_ctx=1,
                          write_state=False, cu_q_host=[0, 1])
        out = self.model.forward(b, self.kv, self.states)
        counts = [n if s.phase == "decode" else (1 if p0 + n == s.n_prompt else 0) for s, p0, n in rows]
        per_owner, where = [0] * W, []
        for (s, _, _), c in zip(rows, counts):
            o = s.owner
            where.append((o, per_owner[o]))
            per_owner[o] += c
        M, V = max(1, max(per_owner)), out.logits.shape[1]
        local = torch.zeros(M, V, dtype=torch.float32, device=self.device)
        if own and per_owner[R]:
            local[:per_owner[R]] = out.logits[:per_owner[R]].float()
        parts = [torch.empty_like(local) for _ in range(W)]
        dist.all_gather(parts, local, group=self.model.pctx.dp_group)
        idx = [o * M + off + j for (o, off), c in zip(where, counts) for j in range(c)]
        logits = torch.cat(parts, 0).index_select(0, torch.tensor(idx, dtype=torch.int64, device=self.device))
        self._stats.dp_gather_bytes = getattr(self._stats, "dp_gather_bytes", 0) + W * M * V * 4
        self._finish_rows(rows, None, logits, None, verify)

    def _masks_ahead(self, rows):
        """Grammar-constrained sequences: the vocabulary mask of the token each of them picks in this step depends
        only on its constraint state, which is already known, so helper threads compute the masks while the forward
        pass runs on the GPU (the engine thread waits for the logits with the interpreter lock released). The
        reference computes them on mask threads the same way (``src/engine/lm/response_format.rs``)."""
        todo = [s for s, p0, n in rows if s.constraint is not None and s.mask_ahead is None
                and (s.phase == "decode" or p0 + n >= s.n_prompt)]
        if not todo:
            return
        if self._mask_pool is None:
            from concurrent.futures import ThreadPoolExecutor
            self._mask_pool = ThreadPoolExecutor(max_workers=4, thread_name_prefix="legion-mask")
        for s in todo:
            s.mask_ahead = self._mask_pool.submit(s.constraint.mask)

    def _take_mask(self, s: Seq):
        if s.constraint is None:
            return None
        fut, s.mask_ahead = s.mask_ahead, None
        if fut is not None:
            self._stats.masks_ahead += 1
            return fut.result()
        return s.constraint.mask()

    def _forward_and_finish(self, rows, verify: bool):
        self._masks_ahead(rows)
        if self.dp_world > 1:
            return self._dp_forward_and_finish(rows, verify)
        all_decode_1 = all(s.phase == "decode" and n == 1 for s, _, n in rows)
        need_hidden = self.drafter is not None and getattr(self.drafter, "needs_hidden", False)
        hm = self._stats.host_ms
        t0 = time.perf_counter()
        if self._graphs is not None and all_decode_1 and not need_hidden:
            picked, logits = self._graphs.run(rows)
            if picked is not None:
                t1 = time.perf_counter()
                hm["forward"] += (t1 - t0) * 1e3
                self._finish_rows(rows, None, logits, None, verify, picked=picked)
                hm["finish"] += (time.perf_counter() - t1) * 1e3
                return
        nvtx = self.cfg.nvtx and self.device.type == "cuda"
        if nvtx:
            torch.cuda.nvtx.range_push(f"step {len(rows)} seqs {sum(r[2] for r in rows)} tokens")
        b = self.build_batch(rows, write_state=not verify)
        if verify and self.hybrid:
            b.replay = {}
        if need_hidden:
            b.capture_layers = getattr(self.drafter, "capture_layers", None)
        t1 = time.perf_counter()
        out = self.model.forward(b, self.kv, self.states)
        if self.step_hook is not None:
            self.step_hook([(s.req.request_id, p0, n, s.phase) for s, p0, n in rows])
        t2 = time.perf_counter()
        self._finish_rows(rows, b, out.logits, out, verify)
        if nvtx:
            torch.cuda.nvtx.range_pop()
        hm["build"] += (t1 - t0) * 1e3
        hm["forward"] += (t2 - t1) * 1e3
        hm["finish"] += (time.perf_counter() - t2) * 1e3

    # ------------------------------------------------------------------ sampling / verification
    def _pick(self, s: Seq, logits_row: torch.Tensor, device_pick: Optional[int] = None) -> Tuple[int, Optional[TokenLogprob]]:
        sp = s.req.sampling
        mask = self._take_mask(s)
        if device_pick is not None and sp.greedy and sp.plain and mask is None:
            return device_pick, None
        tok, lg = s.sampler.sample(logits_row, mask, self.eos_ids if not sp.ignore_eos else (), s.n_out)
        lp = None
        if sp.logprobs:
            v, top = top_logprobs(lg, tok, sp.top_logprobs)
            lp = TokenLogprob(self.tok.decode([tok]), tok, v,
                              [TokenLogprob(self.tok.decode([i]), i, x) for i, x in top])
        return tok, lp

    def _finish_rows(self, rows, b: Optional[StepBatch], logits, out, verify: bool, picked=None):
        r = 0
        commits: List[Tuple[int, int]] = []     # (row index in batch, kept tokens) for replay
        fed = [([s.tokens[-1]] + s.drafts[:n - 1]) if s.phase == "decode" else s.tokens[p0:p0 + n] for s, p0, n in rows]
        step_items = []                          # (seq, first position, fed tokens, kept rows, batch index)
        all_plain = all(s.req.sampling.greedy and s.req.sampling.plain and s.constraint is None for s, _, _ in rows)
        device_picks = picked
        device_accept = None                     # batch index -> (accepted drafts, token after them), from the device
        if device_picks is None and logits is not None and logits.shape[0] and all_plain:
            from .. import ops
            if verify and logits.is_cuda:
                device_accept, device_picks = self._accept_on_device(rows, logits)
            else:
                device_picks = ops.argmax(logits).tolist()
        logits_host = None
        if logits is not None and not all_plain:
            logits_host = logits.float().cpu()
        for bi, (s, p0, n) in enumerate(rows):
            if s.phase == "prefill":
                s.n_computed = p0 + n
                s.table.n_tokens = s.n_computed
                step_items.append((s, p0, fed[bi], n, bi))
                if self.saved is not None and s.n_computed in s.save_points:
                    self._snapshot(s, s.n_computed, "anchor")
                if s.n_computed < s.n_prompt:
                    continue
                # prompt done: cache its full blocks, sample the first token
                if self.radix is not None:
                    self._own_blocks(s)
                    self.radix.insert(s.key_tokens(s.n_prompt), s.table.blocks)
                row = logits_host[r] if logits_host is not None else None
                tok, lp = self._pick(s, row, device_picks[r] if device_picks is not None else None)
                r += 1
                s.phase = "decode"
                if s.first_ms == 0.0:
                    s.first_ms = now_ms()
                    s.usage.prefill_ms = s.first_ms - s.admit_ms
                self._advance(s, [tok], [lp])
                continue
            # decode / verify rows: n = 1 + drafts
            accepted: List[int] = []
            lps: List[Optional[TokenLogprob]] = []
            k = n - 1
            if device_accept is not None and bi in device_accept:
                a, bonus = device_accept[bi]
                accepted = list(s.drafts[:a]) + [bonus]
                lps = [None] * len(accepted)
            for j in range(n if not accepted else 0):
                row = logits_host[r + j] if logits_host is not None else None
                dp = device_picks[r + j] if device_picks is not None else None
                if j < k:
                    ok, tok, lp = self._verify_one(s, row, dp, s.drafts[j])
                    accepted.append(tok)
                    lps.append(lp)
                    if not ok:
                        break
                else:
                    tok, lp = self._pick(s, row, dp)
                    accepted.append(tok)
                    lps.append(lp)
            r += n
            if k:
                if s.spec_state is not None:
                    s.spec_state.update(k, len(accepted) - 1, max(s.spec_cap, k))
                self._stats.spec_draft_tokens += k
                self._stats.spec_accepted_tokens += len(accepted) - 1
                self._stats.spec_verify_steps += 1
                s.usage.draft_tokens += k
                s.usage.accepted_tokens += len(accepted) - 1
            kept = len(accepted)              # rows of this step whose KV / state are valid
            s.n_computed = p0 + kept
            s.table.n_tokens = s.n_computed
            if verify:
                commits.append((bi, kept))
            step_items.append((s, p0, fed[bi], kept, bi))
            self._advance(s, accepted, lps)
        if verify and self.hybrid and b is not None and commits:
            self.model.commit_replay(b, self.states, commits)
        if self.drafter is not None and not self.drafter.model_free:
            if out is not None:
                self.drafter.on_step([it for it in step_items if not it[0].finished], b, out)
            live = [s for s, _, _ in rows if s in self.running and s.phase == "decode"]
            if live and len(live) <= self.cfg.spec_max_batch:
                td = time.perf_counter()
                self.drafter.draft_batch(live, self.cfg.spec_k)
                ms = (time.perf_counter() - td) * 1e3
                self._draft_ms_step += ms
                if self._depth_model is not None:
                    self._depth_model.observe_draft(len(live), self.cfg.spec_k, ms)

    def _accept_on_device(self, rows, logits):
        """Greedy verification without bringing the step's arg-max rows to the host: the arg-max of every logits
        row, then one small kernel that walks each sequence's drafts against them and returns (accepted drafts,
        token after the accepted prefix) per sequence: two integers per sequence come back instead of one per row
        (``csrc/spec.cu``; the reference's device-side accept is ``src/cuda/mtp_cond.cu:33``). Returns
        ({batch index: (accepted, next token)} for the decode rows, per-row picks for prompt rows that end here)."""
        from .. import ops
        dev = logits.device
        groups = []                               # (batch index, first logits row, rows, drafts)
        r = 0
        for bi, (s, p0, n) in enumerate(rows):
            if s.phase == "prefill":
                if p0 + n >= s.n_prompt:
                    groups.append((bi, r, 1, []))
                    r += 1
                continue
            groups.append((bi, r, n, list(s.drafts[:n - 1])))
            r += n
        G = len(groups)
        maxd = max(1, max(len(g[3]) for g in groups))
        host = torch.zeros(G, maxd + 2, dtype=torch.int32)
        for i, (_, r0, _, d) in enumerate(groups):
            host[i, 0], host[i, 1] = r0, len(d)
            if d:
                host[i, 2:2 + len(d)] = torch.tensor(d, dtype=torch.int32)
        packed = host.to(dev, non_blocking=True)
        target = ops.sm100.argmax(logits)
        acc, bonus, _ = ops.sm100.spec_accept(target, packed[:, 0].contiguous(), packed[:, 2:].contiguous(),
                                              packed[:, 1].contiguous())
        res = torch.stack([acc, bonus]).cpu().tolist()
        accept = {}
        picks: List[Optional[int]] = [None] * int(logits.shape[0])
        for i, (bi, r0, n, d) in enumerate(groups):
            if rows[bi][0].phase == "prefill":
                picks[r0] = res[1][i]
            else:
                accept[bi] = (res[0][i], res[1][i])
        return accept, picks

    def _verify_one(self, s: Seq, row, device_pick, draft: int):
        """One draft token against the target's row: greedy = must equal the arg-max; sampled = exact
        rejection sampling against a point-mass draft (accept with probability p(draft), otherwise draw
        from the distribution with the draft removed)."""
        sp = s.req.sampling
        if sp.greedy and sp.plain and device_pick is not None:
            return device_pick == draft, device_pick, None
        mask = self._take_mask(s)
        lg = s.sampler.adjusted(row, mask, self.eos_ids if not sp.ignore_eos else (), s.n_out)
        lp = None
        if sp.greedy:
            tok = int(torch.argmax(lg))
            ok = tok == draft
        else:
            dist = s.sampler.distribution(lg)
            if s.sampler.rng.uniform() < float(dist[draft]):
                tok, ok = draft, True
            else:
                resid = dist.clone()
                resid[draft] = 0
                tok = s.sampler.draw(resid / resid.sum()) if float(resid.sum()) > 0 else draft
                ok = False
        if sp.logprobs:
            v, top = top_logprobs(lg, tok, sp.top_logprobs)
            lp = TokenLogprob(self.tok.decode([tok]), tok, v,
                              [TokenLogprob(self.tok.decode([i]), i, x) for i, x in top])
        return ok, tok, lp

    # ------------------------------------------------------------------ token bookkeeping / streaming
    def _advance(self, s: Seq, toks: List[int], lps, constrained_done: bool = False):
        sp = s.req.sampling
        text_out, ids_out, lp_out = "", [], []
        reason: Optional[FinishReason] = None
        for tok, lp in zip(toks, lps):
            s.tokens.append(tok)
            s.n_out += 1
            s.sampler.accept(tok)
            if s.constraint is not None and not constrained_done:
                s.constraint.advance(tok)
            self._stats.completion_tokens += 1
            s.usage.completion_tokens += 1
            is_eos = (tok in self.eos_ids or tok in sp.stop_token_ids) and not sp.ignore_eos \
                and s.n_out > sp.min_tokens
            if is_eos:
                reason = FinishReason.STOP
                break
            piece = s.detok.push(tok)
            ids_out.append(tok)
            if lp is not None:
                lp_out.append(lp)
            if piece:
                shown = s.stop.push(piece)
                text_out += shown
                if s.stop.hit is not None:
                    reason = FinishReason.STOP_SEQUENCE
                    break
            if s.constraint is not None and s.constraint.finished():
                reason = FinishReason.STOP
                break
            if s.n_out >= sp.max_tokens or len(s.tokens) >= self.cfg.ctx_size:
                reason = FinishReason.LENGTH
                break
        self._emit(s, text_out, ids_out, lp_out)
        if reason is not None:
            # drop tokens generated past the stopping point of a multi-token step
            if reason in (FinishReason.STOP, FinishReason.STOP_SEQUENCE, FinishReason.LENGTH):
                pass
            self._finish(s, reason)

    def _emit(self, s: Seq, text: str, ids: List[int], lps):
        if not text and not ids:
            return
        segments = [("text", text)]
        if s.reason is not None and text:
            segments = s.reason.push(text)
        first = True
        for channel, seg in segments:
            calls = []
            if channel == "text" and s.tools is not None:
                seg, calls = s.tools.push(seg)
            if seg or (first and ids):
                s.stream.put(TokenEvent(kind="reasoning" if channel == "reasoning" else "text", text=seg,
                                        token_ids=ids if first else [], logprobs=lps if first else []))
                first = False
            for call in calls:
                s.stream.put(TokenEvent(kind="tool_call", tool_call=call))
        if first and ids:
            s.stream.put(TokenEvent(kind="text", text="", token_ids=ids, logprobs=lps))

    def _snapshot(self, s: Seq, n_tokens: int, kind: str, tail_block: Optional[int] = None):
        slot, evicted = self.saved.reserve()
        if slot is None:
            return
        if evicted is not None and evicted.tail_block is not None:
            self.pool.decref(evicted.tail_block)
        self.states.copy(s.slot, slot)
        if tail_block is not None:
            self.pool.incref(tail_block)
        self.saved.store(s.key_tokens(), n_tokens, slot, kind, tail_block, on_replace=self._drop_tail_ref)

    def _drop_tail_ref(self, old):
        if old.tail_block is not None:
            self.pool.decref(old.tail_block)

    def _release(self, s: Seq):
        if s.radix_handle is not None and self.radix is not None:
            self.radix.unlock(s.radix_handle)
            s.radix_handle = None
        s.table.free(self.pool)
        if s.slot >= 0:
            self._free_slots.append(s.slot)
            s.slot = -1
        if self.drafter is not None:
            self.drafter.release(s)

    def _finish(self, s: Seq, reason: FinishReason):
        if s.finished:
            return
        s.finished = True
        tail = s.stop.flush() if (s.stop is not None and reason != FinishReason.STOP_SEQUENCE) else ""
        if tail:
            self._emit(s, tail, [], [])
        if s.reason is not None:
            for channel, seg in s.reason.flush():
                s.stream.put(TokenEvent(kind="reasoning" if channel == "reasoning" else "text", text=seg))
        if s.tools is not None:
            seg, calls = s.tools.flush()
            if seg:
                s.stream.put(TokenEvent(kind="text", text=seg))
            for call in calls:
                s.stream.put(TokenEvent(kind="tool_call", tool_call=call))
            if s.tools.calls and reason == FinishReason.STOP:
                reason = FinishReason.TOOL_CALLS
        # end-of-reply save: the computed part of the conversation stays reusable by the next turn
        if reason not in (FinishReason.CANCELLED, FinishReason.ERROR) and s.phase == "decode" and s.slot >= 0:
            n = s.n_computed
            if self.radix is not None:
                self._own_blocks(s)
                self.radix.insert(s.key_tokens(n), s.table.blocks)
            if self.saved is not None and n > 0:
                bs = self.cfg.block_size
                tail_block = s.table.blocks[n // bs] if n % bs and n // bs < len(s.table.blocks) else None
                self._snapshot(s, n, "tail" if n % bs else "anchor", tail_block)
        now = now_ms()
        s.usage.decode_ms = max(0.0, now - (s.first_ms or now))
        if s in self.running:
            self.running.remove(s)
        self._release(s)
        self.waiting.charge(s.key, s.usage.total_tokens)
        s.stream.put(TokenEvent(kind="finished", finish_reason=reason, usage=s.usage))
        self._by_id.pop(s.req.request_id, None)

    # ------------------------------------------------------------------ convenience
    def generate_text(self, prompt=None, tokens=None, **sampling) -> "Completion":
        req = GenerateRequest(prompt=prompt, prompt_tokens=tokens, sampling=SamplingParams(**sampling))
        return self.generate(req).collect()


def build_engine(cfg: ModelConfig, weights=None, engine_cfg: Optional[EngineConfig] = None, tokenizer=None,
                 device="cpu", dtype=None, pctx: Optional[ParallelCtx] = None, seed: int = 0, start: bool = True) -> LmEngine:
    """Random-init (or given) weights -> Decoder -> LmEngine."""
    from ..models.weights import random_weights
    dev = torch.device(device)
    if dtype is None:
        dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    if weights is None:
        weights = random_weights(cfg, dev, dtype, seed=seed)
    ec = engine_cfg or EngineConfig()
    ec.device = str(dev)
    model = Decoder(cfg, weights, pctx, max_position=ec.ctx_size + 8)
    return LmEngine(model, tokenizer or ByteTokenizer(cfg.vocab), ec, start=start)
