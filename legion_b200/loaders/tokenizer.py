"""Tokenizers: byte-level BPE built from GGUF metadata (``tokenizer.ggml.*``) or an HF
``tokenizer.json``, and a plain byte tokenizer for the tiny random-weight test models.

The BPE follows GPT-2's scheme the way llama.cpp applies it (``src/tokenizer.rs:177-762`` in the
reference): regex pre-tokenisation per ``tokenizer.ggml.pre``, bytes mapped to printable code points,
lowest-rank merge first, special tokens matched verbatim before pre-tokenisation.
"""
from __future__ import annotations

import json
import os
from functools import lru_cache
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

try:
    import regex as _re
except ImportError:  # pragma: no cover
    import re as _re


class Tokenizer:
    vocab_size: int = 0
    bos_id: Optional[int] = None
    eos_ids: Tuple[int, ...] = ()
    chat_template: Optional[str] = None
    add_bos: bool = False

    def encode(self, text: str, add_special: bool = False, parse_special: bool = True) -> List[int]:
        raise NotImplementedError

    def decode(self, ids: Sequence[int], skip_special: bool = False) -> str:
        raise NotImplementedError

    def token_bytes(self, tid: int) -> bytes:
        """Raw bytes of one token (used by the grammar matcher)."""
        return self.decode([tid]).encode("utf-8", "ignore")

    def special_token(self, name: str) -> Optional[str]:
        return None

    def token_to_id(self, text: str) -> Optional[int]:
        """Id of the single token ``text`` stands for (special tokens by name), or None."""
        ids = self.encode(text, add_special=False, parse_special=True)
        return ids[0] if len(ids) == 1 else None


class ByteTokenizer(Tokenizer):
    """ids 0..255 are bytes; 256 = <bos>, 257 = <eos>, 258.. = <|im_start|>, <|im_end|>, <think>, </think>,
    <tool_call>, </tool_call>, <|vision_start|>, <|image_pad|>, <|vision_end|>; the rest of the vocabulary is unused
    filler."""

    SPECIALS = ["<bos>", "<eos>", "<|im_start|>", "<|im_end|>", "<think>", "</think>", "<tool_call>", "</tool_call>",
                "<|vision_start|>", "<|image_pad|>", "<|vision_end|>"]

    def __init__(self, vocab_size: int = 4096):
        self.vocab_size = vocab_size
        self.bos_id, self.eos_ids = 256, (257, 259)
        self._sp = {s: 256 + i for i, s in enumerate(self.SPECIALS)}
        self._sp_inv = {v: k for k, v in self._sp.items()}
        self.chat_template = DEFAULT_CHATML_TEMPLATE

    def encode(self, text, add_special=False, parse_special=True):
        ids: List[int] = [self.bos_id] if add_special and self.add_bos else []
        i = 0
        while i < len(text):
            if parse_special and text[i] == "<":
                hit = next((s for s in self.SPECIALS if text.startswith(s, i)), None)
                if hit:
                    ids.append(self._sp[hit])
                    i += len(hit)
                    continue
            ids.extend(text[i].encode("utf-8"))
            i += 1
        return ids

    def decode(self, ids, skip_special=False):
        out = bytearray()
        for t in ids:
            if t < 256:
                out.append(t)
            elif t in self._sp_inv:
                if not skip_special:
                    out.extend(self._sp_inv[t].encode())
            else:
                out.extend(f"<0x{t:X}>".encode())
        return out.decode("utf-8", "replace")

    def token_bytes(self, tid):
        if tid < 256:
            return bytes([tid])
        return self._sp_inv.get(tid, f"<0x{tid:X}>").encode()


@lru_cache(maxsize=1)
def _byte_to_unicode() -> Dict[int, str]:
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


PRE_PATTERNS = {
    "gpt2": r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+",
    "llama3": r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+",
    "qwen2": r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+",
    "deepseek-v3": r"\p{N}{1,3}|[一-龥぀-ゟ゠-ヿ]+|[!\"#$%&'()*+,\-./:;<=>?@\[\\\]^_`{|}~][A-Za-z]+|[^\r\n\p{L}\p{P}\p{S}]?[\p{L}\p{M}]+| ?[\p{P}\p{S}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+",
}
PRE_PATTERNS["default"] = PRE_PATTERNS["gpt2"]
PRE_PATTERNS["qwen35"] = PRE_PATTERNS["qwen2"]


class BpeTokenizer(Tokenizer):
    def __init__(self, tokens: Sequence[str], merges: Sequence[str], pre: str = "gpt2",
                 token_types: Optional[Sequence[int]] = None, bos_id=None, eos_ids=(), add_bos=False,
                 chat_template=None, extra_special: Iterable[str] = (), visible: Iterable[str] = ()):
        """``extra_special``: tokens matched whole in the text and left out of decoded text when special tokens are
        skipped (control tokens). ``visible``: tokens matched whole but always rendered (GGUF's user-defined kind,
        an HF added token with ``special: false``): reasoning and tool-call markers the text parsers must see."""
        self.tokens = list(tokens)
        self.vocab_size = len(self.tokens)
        self.vocab = {t: i for i, t in enumerate(self.tokens)}
        self.ranks = {}
        for r, m in enumerate(merges):
            a, _, b = m.partition(" ")
            self.ranks[(a, b)] = r
        self.pat = _re.compile(PRE_PATTERNS.get(pre, PRE_PATTERNS["default"]))
        self.bos_id, self.eos_ids, self.add_bos, self.chat_template = bos_id, tuple(eos_ids), add_bos, chat_template
        b2u = _byte_to_unicode()
        self._b2u = b2u
        self._u2b = {v: k for k, v in b2u.items()}
        # GGUF token types: 3 = control, 4 = user defined
        sp = set(extra_special)
        vis = set(visible)
        if token_types is not None:
            sp |= {self.tokens[i] for i, t in enumerate(token_types) if t == 3}
            vis |= {self.tokens[i] for i, t in enumerate(token_types) if t == 4}
        sp -= vis
        self.special = {s: self.vocab[s] for s in sp | vis if s in self.vocab}
        self._special_ids = set(self.special.values())
        self._hidden_ids = {self.vocab[s] for s in sp if s in self.vocab}
        self._sp_re = None
        if self.special:
            alts = sorted(self.special, key=len, reverse=True)
            self._sp_re = _re.compile("|".join(_re.escape(a) for a in alts))
        self._cache: Dict[str, List[int]] = {}
        # the merge loop runs in the native host runtime when it is built (same procedure, same result)
        self._native = None
        from ..kv.blocks import NATIVE
        if NATIVE is not None and hasattr(NATIVE, "BpeMerger") and all(" " not in t for t in self.tokens):
            self._native = NATIVE.BpeMerger(self.tokens, [tuple(k) for k in self.ranks])

    def _bpe(self, word: str) -> List[int]:
        hit = self._cache.get(word)
        if hit is not None:
            return hit
        if self._native is not None:
            ids = self._native.encode_word(word)
            if len(self._cache) < 65536:
                self._cache[word] = ids
            return ids
        parts = list(word)
        while len(parts) > 1:
            best, bi = None, -1
            for i in range(len(parts) - 1):
                r = self.ranks.get((parts[i], parts[i + 1]))
                if r is not None and (best is None or r < best):
                    best, bi = r, i
            if best is None:
                break
            parts[bi:bi + 2] = [parts[bi] + parts[bi + 1]]
        ids = []
        for p in parts:
            t = self.vocab.get(p)
            if t is None:   # unknown piece: fall back to its bytes' single-symbol tokens
                ids.extend(self.vocab[c] for c in p if c in self.vocab)
            else:
                ids.append(t)
        if len(self._cache) < 65536:
            self._cache[word] = ids
        return ids

    PARALLEL_CHARS = 32768          # texts from this length on encode their pre-tokens on several threads
    PARALLEL_THREADS = 8

    def _encode_plain(self, text: str) -> List[int]:
        if (len(text) >= self.PARALLEL_CHARS and self._native is not None and hasattr(self._native, "encode_pieces")):
            return self._encode_parallel(text)
        out: List[int] = []
        for m in self.pat.finditer(text):
            word = "".join(self._b2u[b] for b in m.group(0).encode("utf-8"))
            out.extend(self._bpe(word))
        return out

    def _encode_parallel(self, text: str) -> List[int]:
        """Long prompts: the pre-tokeniser's pattern cuts the text once, then contiguous runs of the pieces are mapped
        and merged by the native runtime on several threads (it runs without the interpreter lock); the runs' ids are
        joined in order, so the result is that of the serial loop."""
        from concurrent.futures import ThreadPoolExecutor
        pieces = [m.group(0).encode("utf-8") for m in self.pat.finditer(text)]
        n = max(1, min(self.PARALLEL_THREADS, os.cpu_count() or 1, len(pieces) // 1024 or 1))
        per = (len(pieces) + n - 1) // n
        runs = [pieces[i:i + per] for i in range(0, len(pieces), per)]
        if len(runs) == 1:
            return list(self._native.encode_pieces(runs[0]))
        with ThreadPoolExecutor(len(runs)) as ex:
            parts = list(ex.map(self._native.encode_pieces, runs))
        out: List[int] = []
        for p in parts:
            out.extend(p)
        return out

    def encode(self, text, add_special=False, parse_special=True):
        ids: List[int] = [self.bos_id] if (add_special and self.add_bos and self.bos_id is not None) else []
        if parse_special and self._sp_re is not None:
            pos = 0
            for m in self._sp_re.finditer(text):
                if m.start() > pos:
                    ids.extend(self._encode_plain(text[pos:m.start()]))
                ids.append(self.special[m.group(0)])
                pos = m.end()
            if pos < len(text):
                ids.extend(self._encode_plain(text[pos:]))
        else:
            ids.extend(self._encode_plain(text))
        return ids

    def token_bytes(self, tid):
        t = self.tokens[tid]
        if tid in self._special_ids:
            return t.encode("utf-8")
        return bytes(self._u2b.get(c, ord("?")) for c in t)

    def decode(self, ids, skip_special=False):
        out = bytearray()
        for t in ids:
            if t < 0 or t >= self.vocab_size:
                continue
            if t in self._special_ids:
                if not (skip_special and t in self._hidden_ids):
                    out.extend(self.tokens[t].encode("utf-8"))
            else:
                out.extend(self.token_bytes(t))
        return out.decode("utf-8", "replace")

    @classmethod
    def from_gguf_metadata(cls, md: dict) -> "BpeTokenizer":
        eos = [md[k] for k in ("tokenizer.ggml.eos_token_id", "tokenizer.ggml.eot_token_id") if k in md]
        return cls(md["tokenizer.ggml.tokens"], md.get("tokenizer.ggml.merges", []),
                   pre=md.get("tokenizer.ggml.pre", "gpt2"), token_types=md.get("tokenizer.ggml.token_type"),
                   bos_id=md.get("tokenizer.ggml.bos_token_id"), eos_ids=eos,
                   add_bos=bool(md.get("tokenizer.ggml.add_bos_token", False)),
                   chat_template=md.get("tokenizer.chat_template"))

    @classmethod
    def from_hf_dir(cls, path: str) -> "BpeTokenizer":
        tj = json.load(open(os.path.join(path, "tokenizer.json"), encoding="utf-8"))
        model = tj["model"]
        vocab = model["vocab"]
        added = {a["content"]: a["id"] for a in tj.get("added_tokens", [])}
        shown = [a["content"] for a in tj.get("added_tokens", []) if not a.get("special", True)]
        size = max(list(vocab.values()) + list(added.values())) + 1
        tokens = [f"<unused{i}>" for i in range(size)]
        for t, i in vocab.items():
            tokens[i] = t
        for t, i in added.items():
            tokens[i] = t
        merges = [m if isinstance(m, str) else " ".join(m) for m in model.get("merges", [])]
        cfg = {}
        tc = os.path.join(path, "tokenizer_config.json")
        if os.path.exists(tc):
            cfg = json.load(open(tc, encoding="utf-8"))
        def tok_id(name):
            v = cfg.get(name)
            if isinstance(v, dict):
                v = v.get("content")
            return added.get(v, vocab.get(v)) if v else None
        eos = [i for i in [tok_id("eos_token")] if i is not None]
        if cls is BpeTokenizer and model.get("byte_fallback") and "ByteLevel" not in json.dumps(tj.get("pre_tokenizer")):
            # raw-text BPE with byte tokens (the Gemma family): special tokens are the added ones marked special
            for t in ("<end_of_turn>", "<turn|>"):
                if t in added and added[t] not in eos:
                    eos.append(added[t])
            return Gemma4Tokenizer(tokens, merges, bos_id=tok_id("bos_token"), eos_ids=eos,
                                   chat_template=cfg.get("chat_template"), extra_special=added.keys(), visible=shown)
        tok = cls(tokens, merges, pre="qwen2", bos_id=tok_id("bos_token"), eos_ids=eos,
                  chat_template=cfg.get("chat_template"), extra_special=added.keys(), visible=shown)
        pat = _hf_pre_pattern(tj.get("pre_tokenizer"))
        if pat is not None:
            tok.pat = pat
        return tok


def _hf_pre_pattern(pre):
    """The cut pattern a ``tokenizer.json`` pre-tokeniser describes: the regex of its ``Split`` step, or GPT-2's when
    a ``ByteLevel`` step does the cutting itself; None when there is none to read (the family default stays)."""
    steps = pre.get("pretokenizers", [pre]) if isinstance(pre, dict) else []
    for st in steps:
        if st.get("type") == "Split" and isinstance(st.get("pattern"), dict) and st["pattern"].get("Regex"):
            try:
                return _re.compile(st["pattern"]["Regex"])
            except Exception:
                return None
    for st in steps:
        if st.get("type") == "ByteLevel" and st.get("use_regex", True):
            return _re.compile(PRE_PATTERNS["gpt2"])
    return None


class Gemma4Tokenizer(BpeTokenizer):
    """Gemma 4's vocabulary (``tokenizer.ggml.model = "gemma4"``; an HF ``tokenizer.json`` whose BPE model has
    ``byte_fallback``): merge-rank BPE over the text's own characters, not over the GPT-2 byte alphabet. The text is
    cut into runs of newlines and runs of everything else; a newline run that is a token is taken whole; elsewhere
    spaces become U+2581 and the run is merged by rank; a piece no token covers falls back to its ``<0xXX>`` byte
    tokens. A begin-of-sequence token is always added.

    Reference counterpart: ``src/tokenizer/gemma4.rs`` (the rules of llama.cpp's ``LLAMA_VOCAB_PRE_TYPE_GEMMA4``)."""
    SPACE = "\u2581"

    # markers the chat parsers read: always rendered (the reference's converter marks them user-defined)
    VISIBLE = ("<|channel>", "<channel|>", "<|tool_call>", "<tool_call|>", "<|tool_response>", "<tool_response|>",
               '<|"|>')

    def __init__(self, tokens, merges, token_types=None, bos_id=None, eos_ids=(), chat_template=None,
                 extra_special: Iterable[str] = (), visible: Iterable[str] = ()):
        super().__init__(tokens, merges, pre="gpt2", token_types=token_types, bos_id=bos_id, eos_ids=eos_ids,
                         add_bos=True, chat_template=chat_template, extra_special=extra_special,
                         visible=tuple(visible) + self.VISIBLE)
        self.pat = _re.compile(r"[^\n]+|\n+")
        tt = list(token_types) if token_types is not None else [1] * len(self.tokens)
        self.byte_id: Dict[int, int] = {}
        for i, t in enumerate(self.tokens):
            if (tt[i] == 6 or token_types is None) and len(t) == 6 and t.startswith("<0x") and t.endswith(">"):
                try:
                    self.byte_id[int(t[3:5], 16)] = i
                except ValueError:
                    pass
        self._byte_of = {i: b for b, i in self.byte_id.items()}
        # byte tokens are pieces of text, never markers: not matched by name, rendered as their byte
        self.special = {t: i for t, i in self.special.items() if i not in self._byte_of}
        self._special_ids = set(self.special.values())
        self._hidden_ids &= self._special_ids
        self._sp_re = None
        if self.special:
            self._sp_re = _re.compile("|".join(_re.escape(a) for a in sorted(self.special, key=len, reverse=True)))

    def _fallback(self, piece: str) -> List[int]:
        return [self.byte_id[b] for b in piece.encode("utf-8") if b in self.byte_id]

    def _bpe(self, word: str) -> List[int]:
        hit = self._cache.get(word)
        if hit is not None:
            return hit
        if self._native is not None and all(c in self.vocab for c in word):
            ids = list(self._native.encode_word(word))
        else:
            parts = list(word)
            while len(parts) > 1:
                best, bi = None, -1
                for i in range(len(parts) - 1):
                    r = self.ranks.get((parts[i], parts[i + 1]))
                    if r is not None and (best is None or r < best):
                        best, bi = r, i
                if best is None:
                    break
                parts[bi:bi + 2] = [parts[bi] + parts[bi + 1]]
            ids = []
            for p_ in parts:
                t = self.vocab.get(p_)
                if t is None:
                    ids.extend(self._fallback(p_))
                else:
                    ids.append(t)
        if len(self._cache) < 65536:
            self._cache[word] = ids
        return ids

    def _encode_plain(self, text: str) -> List[int]:
        out: List[int] = []
        for m in self.pat.finditer(text):
            word = m.group(0)
            if word[0] == "\n":
                t = self.vocab.get(word)
                if t is not None:
                    out.append(t)
                    continue
            out.extend(self._bpe(word.replace(" ", self.SPACE)))
        return out

    def token_bytes(self, tid):
        if tid in self._byte_of:
            return bytes([self._byte_of[tid]])
        t = self.tokens[tid]
        if tid in self._special_ids:
            return t.encode("utf-8")
        return t.replace(self.SPACE, " ").encode("utf-8")

    @classmethod
    def from_gguf_metadata(cls, md: dict) -> "Gemma4Tokenizer":
        eos = [md[k] for k in ("tokenizer.ggml.eos_token_id", "tokenizer.ggml.eot_token_id") if k in md]
        return cls(md["tokenizer.ggml.tokens"], md.get("tokenizer.ggml.merges", []),
                   token_types=md.get("tokenizer.ggml.token_type"), bos_id=md.get("tokenizer.ggml.bos_token_id"),
                   eos_ids=eos, chat_template=md.get("tokenizer.chat_template"))


class SpmTokenizer(Tokenizer):
    """SentencePiece-style vocabulary as GGUF files of the llama / gemma families carry it (``tokenizer.ggml.model =
    "llama"``): pieces with scores, spaces written as U+2581, byte tokens ``<0xXX>`` for what no piece covers.
    Encoding is the score-ordered bigram merge over the text's characters (the pair whose concatenation is the
    best-scoring piece merges first), as llama.cpp's SPM tokenizer does it; control pieces are matched as text when
    ``parse_special``.

    Reference counterpart: ``src/tokenizer/spm.rs`` (gemma4 tokenizer)."""
    SPACE = "\u2581"

    def __init__(self, tokens: Sequence[str], scores: Sequence[float], token_types: Optional[Sequence[int]] = None,
                 bos_id=None, eos_ids=(), add_bos=True, add_space_prefix=True, chat_template=None):
        import heapq
        self._heapq = heapq
        self.tokens = list(tokens)
        self.scores = list(scores) if scores else [0.0] * len(self.tokens)
        self.vocab_size = len(self.tokens)
        self.vocab = {t: i for i, t in enumerate(self.tokens)}
        tt = list(token_types) if token_types is not None else [1] * len(self.tokens)
        self.token_types = tt
        self.bos_id, self.eos_ids, self.add_bos, self.chat_template = bos_id, tuple(eos_ids), add_bos, chat_template
        self.add_space_prefix = add_space_prefix
        self.byte_id = {}
        for i, t in enumerate(self.tokens):
            if tt[i] == 6 or (len(t) == 6 and t.startswith("<0x") and t.endswith(">")):
                try:
                    self.byte_id[int(t[3:5], 16)] = i
                except ValueError:
                    pass
        self.unk_id = next((i for i, k in enumerate(tt) if k == 2), 0)
        self.special = {self.tokens[i]: i for i, k in enumerate(tt) if k in (3, 4)}
        self._special_ids = set(self.special.values())
        self._sp_re = None
        if self.special:
            alts = sorted(self.special, key=len, reverse=True)
            self._sp_re = _re.compile("|".join(_re.escape(a) for a in alts))

    def _encode_plain(self, text: str) -> List[int]:
        if not text:
            return []
        heapq = self._heapq
        sym = list(text)
        n = len(sym)
        prev = list(range(-1, n - 1))
        nxt = list(range(1, n + 1))
        nxt[-1] = -1
        alive = [True] * n
        heap = []

        def push(a, b):
            if a < 0 or b < 0:
                return
            piece = sym[a] + sym[b]
            i = self.vocab.get(piece)
            if i is not None and self.token_types[i] not in (3,):
                heapq.heappush(heap, (-self.scores[i], a, b, piece))

        for a in range(n - 1):
            push(a, a + 1)
        while heap:
            _, a, b, piece = heapq.heappop(heap)
            if not (alive[a] and alive[b]) or nxt[a] != b or sym[a] + sym[b] != piece:
                continue
            sym[a] = piece
            alive[b] = False
            nxt[a] = nxt[b]
            if nxt[b] >= 0:
                prev[nxt[b]] = a
            push(prev[a], a)
            push(a, nxt[a])
        out: List[int] = []
        i = 0
        while i >= 0:
            piece = sym[i]
            tid = self.vocab.get(piece)
            if tid is not None:
                out.append(tid)
            else:
                for byte in piece.encode("utf-8"):
                    out.append(self.byte_id.get(byte, self.unk_id))
            i = nxt[i]
        return out

    def encode(self, text, add_special=False, parse_special=True):
        ids: List[int] = [self.bos_id] if (add_special and self.add_bos and self.bos_id is not None) else []
        parts = [(False, text)]
        if parse_special and self._sp_re is not None:
            parts, pos = [], 0
            for m in self._sp_re.finditer(text):
                if m.start() > pos:
                    parts.append((False, text[pos:m.start()]))
                parts.append((True, m.group(0)))
                pos = m.end()
            if pos < len(text):
                parts.append((False, text[pos:]))
        prev_special = True            # text at the start, and text right after a control piece, takes the space prefix
        for is_sp, chunk in parts:
            if is_sp:
                ids.append(self.special[chunk])
            else:
                if prev_special and self.add_space_prefix:
                    chunk = " " + chunk
                ids.extend(self._encode_plain(chunk.replace(" ", self.SPACE)))
            prev_special = is_sp
        return ids

    def token_bytes(self, tid):
        t = self.tokens[tid]
        if tid in self._special_ids:
            return b""
        if tid in self.byte_id.values() and t.startswith("<0x"):
            return bytes([int(t[3:5], 16)])
        return t.replace(self.SPACE, " ").encode("utf-8")

    def decode(self, ids, skip_special=False):
        out = bytearray()
        for i in ids:
            if i in self._special_ids:
                if not skip_special:
                    out += self.tokens[i].encode("utf-8")
                continue
            out += self.token_bytes(i)
        s = out.decode("utf-8", "replace")
        return s[1:] if (self.add_space_prefix and s.startswith(" ")) else s

    @classmethod
    def from_gguf_metadata(cls, md: dict) -> "SpmTokenizer":
        eos = [md[k] for k in ("tokenizer.ggml.eos_token_id", "tokenizer.ggml.eot_token_id") if k in md]
        return cls(md["tokenizer.ggml.tokens"], md.get("tokenizer.ggml.scores", []),
                   token_types=md.get("tokenizer.ggml.token_type"), bos_id=md.get("tokenizer.ggml.bos_token_id"),
                   eos_ids=eos, add_bos=bool(md.get("tokenizer.ggml.add_bos_token", True)),
                   add_space_prefix=bool(md.get("tokenizer.ggml.add_space_prefix", True)),
                   chat_template=md.get("tokenizer.chat_template"))


def tokenizer_from_gguf_metadata(md: dict) -> Tokenizer:
    """The tokenizer a GGUF file describes: score-merged pieces (``llama``: llama / gemma families) or byte-level BPE
    with merge ranks (``gpt2``: qwen, deepseek, llama-3)."""
    if md.get("tokenizer.ggml.model", "gpt2") == "llama":
        return SpmTokenizer.from_gguf_metadata(md)
    if md.get("tokenizer.ggml.model") == "gemma4":
        return Gemma4Tokenizer.from_gguf_metadata(md)
    return BpeTokenizer.from_gguf_metadata(md)


DEFAULT_CHATML_TEMPLATE = (
    "{%- if tools %}{{- '<|im_start|>system\\n' }}{%- if messages[0].role == 'system' %}{{- messages[0].content + '\\n\\n' }}{%- endif %}"
    "{{- '# Tools\\n\\nYou may call one or more functions to assist with the user query.\\n\\n<tools>' }}"
    "{%- for tool in tools %}{{- '\\n' }}{{- tool | tojson }}{%- endfor %}"
    "{{- '\\n</tools>\\n\\nFor each function call, return a json object with function name and arguments within "
    "<tool_call></tool_call> XML tags:\\n<tool_call>\\n{\"name\": <function-name>, \"arguments\": <args-json-object>}\\n</tool_call><|im_end|>\\n' }}"
    "{%- else %}{%- if messages[0].role == 'system' %}{{- '<|im_start|>system\\n' + messages[0].content + '<|im_end|>\\n' }}{%- endif %}{%- endif %}"
    "{%- for message in messages %}"
    "{%- if message.role == 'user' or (message.role == 'system' and not loop.first) %}{{- '<|im_start|>' + message.role + '\\n' + message.content + '<|im_end|>\\n' }}"
    "{%- elif message.role == 'assistant' %}{{- '<|im_start|>assistant\\n' }}{%- if message.content %}{{- message.content }}{%- endif %}"
    "{%- if message.tool_calls %}{%- for tc in message.tool_calls %}{{- '\\n<tool_call>\\n{\"name\": \"' + tc.function.name + '\", \"arguments\": ' }}"
    "{{- tc.function.arguments if tc.function.arguments is string else tc.function.arguments | tojson }}{{- '}\\n</tool_call>' }}{%- endfor %}{%- endif %}{{- '<|im_end|>\\n' }}"
    "{%- elif message.role == 'tool' %}{{- '<|im_start|>user\\n<tool_response>\\n' + message.content + '\\n</tool_response><|im_end|>\\n' }}"
    "{%- endif %}{%- endfor %}"
    "{%- if add_generation_prompt %}{{- '<|im_start|>assistant\\n' }}{%- if enable_thinking is defined and enable_thinking is false %}{{- '<think>\\n\\n</think>\\n\\n' }}{%- endif %}{%- endif %}"
)
