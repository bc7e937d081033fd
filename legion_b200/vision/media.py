"""Images in a sequence's token stream: where each image's tokens are, their input rows, the rotary positions they and
the text after them take, and the ids that stand for them in prefix-cache keys.

A chat template writes one placeholder token per image part (between the vision start / end markers); the
placeholder becomes as many tokens as the tower gives rows for that image. Multi-section rotary positions (M-RoPE):
text tokens take one running position on all three axes; an image's tokens take (start, start + row, start +
column) and the text after it continues from start + max(rows, columns), so positions after an image run behind the
token index by a constant ``rope_delta``. Prefix-cache keys must tell two images apart although their tokens carry
the same placeholder id: the key ids of an image's tokens are derived from the image's hash.

Reference counterparts: ``src/model/core/media.rs`` (image tokens, input rows, M-RoPE positions),
``src/engine/lm/vision.rs`` (prefix key)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

from .cache import RowCache, image_hash
from .preprocess import VisionHparams, decode_image, preprocess
from .tower import ImageEmbedding, VisionTower

KEY_MOD = (1 << 31) - 1      # key ids of image tokens are negative 32-bit numbers; vocabulary ids never are


@dataclass
class SeqMedia:
    n_prompt: int
    spans: List[Tuple[int, int]]                   # (first prompt position, tokens) per image
    grids: List[Tuple[int, int, int]]              # (t, h, w) in tokens per image
    rows: Optional[torch.Tensor] = None            # [sum tokens, hidden] input rows, images back to back
    deepstack: List[torch.Tensor] = field(default_factory=list)
    pending: Optional[list] = None                 # per image: (hash, cached embedding or None, patches or None)
    key_ids: List[int] = field(default_factory=list)
    pos3: Optional[torch.Tensor] = None            # [3, n_prompt] int64 rotary positions (multi-section models)
    rope_delta: int = 0
    row_of_pos: Optional[torch.Tensor] = None      # [n_prompt] int64 row of ``rows`` or -1

    def key_tokens(self, tokens: Sequence[int]) -> List[int]:
        out = list(tokens)
        i = 0
        for p0, n in self.spans:
            out[p0:p0 + n] = self.key_ids[i:i + n]
            i += n
        return out

    def materialize(self, rt: "VisionRuntime", device, dtype) -> None:
        """Runs the tower on the images that were not in the row cache and lays the rows out back to back. The
        engine calls this on its own thread when the sequence is placed (the thread that owns the device's stream
        and graph captures); ``attach`` on the caller's thread only decodes and cuts patches."""
        if self.rows is not None or self.pending is None:
            return
        embs = []
        for key, emb, pre in self.pending:
            if emb is None:
                emb = rt.cache.get(key)
            if emb is None:
                emb = rt.tower.encode(pre.patches, pre.grid)
                rt.cache.put(key, emb)
                rt.encoded += 1
            embs.append(emb)
        self.rows = torch.cat([e.rows for e in embs], 0).to(device=device, dtype=dtype)
        n_deep = min((len(e.deepstack) for e in embs), default=0)
        self.deepstack = [torch.cat([e.deepstack[j] for e in embs], 0).to(device=device, dtype=dtype)
                          for j in range(n_deep)]
        self.pending = None

    def rope_position(self, p: int) -> int:
        """Temporal-axis rotary position of token index ``p`` (the only axis for tokens after the prompt)."""
        if self.pos3 is None:
            return p
        if p < self.n_prompt:
            return int(self.pos3[0, p])
        return p + self.rope_delta


def expand_image_tokens(tokens: Sequence[int], image_token: int, counts: Sequence[int],
                        start_token: Optional[int] = None, end_token: Optional[int] = None):
    """Replaces the i-th run of ``image_token`` placeholders by ``counts[i]`` of them. A prompt without placeholders
    gets the images in front (behind a leading BOS-like first token when there is more than one token), wrapped in
    the start / end markers when the vocabulary has them. Returns (tokens, spans)."""
    out: List[int] = []
    spans: List[Tuple[int, int]] = []
    i, k = 0, 0
    n = len(tokens)
    runs = 0
    j = 0
    while j < n:
        if tokens[j] == image_token:
            runs += 1
            while j < n and tokens[j] == image_token:
                j += 1
        else:
            j += 1
    if runs == 0:
        head = list(tokens[:1]) if n > 1 else []
        out.extend(head)
        for c in counts:
            if start_token is not None:
                out.append(start_token)
            spans.append((len(out), c))
            out.extend([image_token] * c)
            if end_token is not None:
                out.append(end_token)
        out.extend(tokens[len(head):])
        return out, spans
    if runs != len(counts):
        raise ValueError(f"the prompt has {runs} image placeholders for {len(counts)} images")
    while i < n:
        if tokens[i] == image_token:
            while i < n and tokens[i] == image_token:
                i += 1
            spans.append((len(out), counts[k]))
            out.extend([image_token] * counts[k])
            k += 1
        else:
            out.append(tokens[i])
            i += 1
    return out, spans


def mrope_positions(n_prompt: int, spans: Sequence[Tuple[int, int]], grids: Sequence[Tuple[int, int, int]]):
    """([3, n_prompt] positions on the (temporal, row, column) axes, rope_delta)."""
    pos = torch.zeros(3, n_prompt, dtype=torch.int64)
    nxt, p = 0, 0
    for (p0, n), (t, gh, gw) in zip(spans, grids):
        if t * gh * gw != n:
            raise ValueError("image span does not match its grid")
        if p0 > p:
            pos[:, p:p0] = torch.arange(nxt, nxt + p0 - p)
            nxt += p0 - p
        tt = torch.arange(t).view(t, 1, 1).expand(t, gh, gw).reshape(-1)
        rr = torch.arange(gh).view(1, gh, 1).expand(t, gh, gw).reshape(-1)
        cc = torch.arange(gw).view(1, 1, gw).expand(t, gh, gw).reshape(-1)
        pos[0, p0:p0 + n] = nxt + tt
        pos[1, p0:p0 + n] = nxt + rr
        pos[2, p0:p0 + n] = nxt + cc
        nxt += max(t, gh, gw)
        p = p0 + n
    if p < n_prompt:
        pos[:, p:] = torch.arange(nxt, nxt + n_prompt - p)
        nxt += n_prompt - p
    return pos, nxt - n_prompt


def mrope_axis_of_freq(half: int, sections: Sequence[int], interleaved: bool) -> torch.Tensor:
    """Axis (0 temporal, 1 row, 2 column) that rotary frequency i of ``half`` turns with. Interleaved layout: the
    axes alternate t, h, w, t, h, w, ... while an axis still has frequencies left, the rest is temporal; sectioned
    layout: the first sections[0] frequencies are temporal, the next sections[1] rows, then columns."""
    ax = torch.zeros(half, dtype=torch.int64)
    if interleaved:
        for a in (1, 2):
            idx = torch.arange(a, min(half, 3 * sections[a]), 3)
            ax[idx] = a
    else:
        s0, s1 = sections[0], sections[0] + sections[1]
        ax[s0:s1] = 1
        ax[s1:s1 + sections[2]] = 2
    return ax


class VisionRuntime:
    """A tower with its preprocessing parameters, the placeholder token ids and the row cache: what an engine needs
    to accept images."""

    def __init__(self, tower: VisionTower, hp: Optional[VisionHparams] = None, image_token: int = -1,
                 start_token: Optional[int] = None, end_token: Optional[int] = None, cache_bytes: int = 256 << 20):
        c = tower.cfg
        self.tower = tower
        self.hp = hp or VisionHparams(patch_size=c.patch_size, spatial_merge_size=c.spatial_merge_size,
                                      temporal_patch_size=c.temporal_patch_size,
                                      resize="stretch" if c.projector == "pool" else "pad")
        self.image_token, self.start_token, self.end_token = image_token, start_token, end_token
        self.cache = RowCache(cache_bytes)
        self.encoded = 0

    def bind_tokenizer(self, tok) -> None:
        """Looks the placeholder and marker ids up in the vocabulary (Qwen and Gemma spellings)."""
        def find(*names):
            for nme in names:
                i = tok.token_to_id(nme) if hasattr(tok, "token_to_id") else None
                if i is not None and i >= 0:
                    return i
            return None
        if self.image_token < 0:
            i = find("<|image_pad|>", "<image_soft_token>", "<|image|>", "<image>")
            if i is None:
                raise ValueError("the vocabulary has no image placeholder token")
            self.image_token = i
        if self.start_token is None:
            self.start_token = find("<|vision_start|>", "<start_of_image>", "<|image>")
        if self.end_token is None:
            self.end_token = find("<|vision_end|>", "<end_of_image>", "<image|>")

    def encode(self, data: bytes) -> Tuple[bytes, ImageEmbedding]:
        key = image_hash(data)
        hit = self.cache.get(key)
        if hit is not None:
            return key, hit
        pre = preprocess(decode_image(data), self.hp)
        emb = self.tower.encode(pre.patches, pre.grid)
        self.cache.put(key, emb)
        self.encoded += 1
        return key, emb

    def attach(self, tokens: Sequence[int], images: Sequence[bytes], hidden: int, mrope: bool):
        """(prompt tokens with the placeholders expanded, SeqMedia). Decoding, resizing and patch cutting happen
        here; the tower itself runs in ``SeqMedia.materialize``."""
        if self.image_token < 0:
            raise ValueError("vision runtime is not bound to a tokenizer")
        if self.tower.cfg.out_hidden != hidden:
            raise ValueError(f"the vision tower gives rows of width {self.tower.cfg.out_hidden}, the model takes {hidden}")
        m = self.hp.spatial_merge_size
        pending, counts, grids, keys = [], [], [], []
        for data in images:
            key = image_hash(data)
            emb = self.cache.get(key)
            if emb is not None:
                pending.append((key, emb, None))
                grid = emb.grid
            else:
                pre = preprocess(decode_image(data), self.hp)
                pending.append((key, None, pre))
                grid = (pre.grid[0], pre.grid[1] // m, pre.grid[2] // m)
            grids.append(grid)
            counts.append(grid[0] * grid[1] * grid[2])
            keys.append(key)
        toks, spans = expand_image_tokens(tokens, self.image_token, counts, self.start_token, self.end_token)
        key_ids: List[int] = []
        for k, c in zip(keys, counts):
            base = int.from_bytes(k[:8], "little")
            key_ids.extend(-1 - ((base + i * 0x9E3779B1) % KEY_MOD) for i in range(c))
        sm = SeqMedia(len(toks), spans, grids, key_ids=key_ids, pending=pending)
        sm.row_of_pos = torch.full((len(toks),), -1, dtype=torch.int64)
        r = 0
        for p0, n in spans:
            sm.row_of_pos[p0:p0 + n] = torch.arange(r, r + n)
            r += n
        if mrope:
            sm.pos3, sm.rope_delta = mrope_positions(len(toks), spans, sm.grids)
        return toks, sm
