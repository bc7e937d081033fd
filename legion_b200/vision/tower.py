"""The vision tower: patches of one image -> input rows of the language model.

Qwen3-VL form (``projector="qwen3vl_merger"``, the tower of Qwen3.5 / Qwen3.6 checkpoints and of ``clip`` mmproj
files with that projector; reference ``src/vision/qwen3vl.rs``, ``src/vision/gpu.rs``): patch embedding (the 3-D
convolution over [3, temporal, patch, patch] is a matrix product over the flattened patch), learned position
embeddings resampled bilinearly from their square table to the image's patch grid, pre-norm ViT blocks (LayerNorm,
biased qkv, two-dimensional rotary embedding over (row, column), unmasked attention, biased output projection,
GELU MLP), then the merger: LayerNorm, the ``merge x merge`` neighbouring patches concatenated, two-layer MLP to the
language model's width. "Deepstack" mergers read the hidden states after chosen blocks and give extra rows that the
language model adds to its residual stream after its first layers.

Pooling form (``projector="pool"``, Gemma-4 style; reference ``src/vision/gemma4v.rs``): same trunk without rotary
embedding, ``merge x merge`` average pool, RMS norm, one projection.

Patches arrive in merge order (``preprocess``), so a token's patches are consecutive rows. Weights are a flat dict
with the names of ``random_vision_weights``; ``loaders.vision`` maps checkpoint names to them."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F


@dataclass
class VisionConfig:
    depth: int = 2
    hidden: int = 32
    n_head: int = 2
    intermediate: int = 64
    out_hidden: int = 64               # width of the language model
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    num_pos: int = 16                  # rows of the learned position table (a square grid)
    deepstack_layers: Tuple[int, ...] = ()
    projector: str = "qwen3vl_merger"  # | "pool"
    act: str = "gelu_tanh"             # | "gelu" | "silu"
    ln_eps: float = 1e-6
    rope_theta: float = 10000.0

    @property
    def head_dim(self) -> int:
        return self.hidden // self.n_head

    @property
    def patch_dim(self) -> int:
        return 3 * self.temporal_patch_size * self.patch_size * self.patch_size


def random_vision_weights(cfg: VisionConfig, device="cpu", dtype=torch.float32, seed: int = 0, std: float = 0.05):
    g = torch.Generator().manual_seed(seed)

    def r(*shape):
        return (torch.randn(*shape, generator=g) * std).to(device=device, dtype=dtype)

    def ones(n):
        return torch.ones(n, device=device, dtype=dtype)

    w: Dict[str, torch.Tensor] = {"patch.w": r(cfg.hidden, cfg.patch_dim), "patch.b": r(cfg.hidden),
                                  "pos": r(cfg.num_pos, cfg.hidden)}
    for i in range(cfg.depth):
        p = f"blk{i}"
        w[f"{p}.ln1.w"], w[f"{p}.ln1.b"] = ones(cfg.hidden), r(cfg.hidden)
        w[f"{p}.qkv.w"], w[f"{p}.qkv.b"] = r(3 * cfg.hidden, cfg.hidden), r(3 * cfg.hidden)
        w[f"{p}.proj.w"], w[f"{p}.proj.b"] = r(cfg.hidden, cfg.hidden), r(cfg.hidden)
        w[f"{p}.ln2.w"], w[f"{p}.ln2.b"] = ones(cfg.hidden), r(cfg.hidden)
        w[f"{p}.fc1.w"], w[f"{p}.fc1.b"] = r(cfg.intermediate, cfg.hidden), r(cfg.intermediate)
        w[f"{p}.fc2.w"], w[f"{p}.fc2.b"] = r(cfg.hidden, cfg.intermediate), r(cfg.hidden)
    m2 = cfg.spatial_merge_size ** 2
    if cfg.projector == "pool":
        w["proj.norm.w"] = ones(cfg.hidden)
        w["proj.w"] = r(cfg.out_hidden, cfg.hidden)
    else:
        names = ["merger"] + [f"ds{j}" for j in range(len(cfg.deepstack_layers))]
        for n in names:
            ln = cfg.hidden if n == "merger" else cfg.hidden * m2
            w[f"{n}.ln.w"], w[f"{n}.ln.b"] = ones(ln), r(ln)
            w[f"{n}.fc1.w"], w[f"{n}.fc1.b"] = r(cfg.hidden * m2, cfg.hidden * m2), r(cfg.hidden * m2)
            w[f"{n}.fc2.w"], w[f"{n}.fc2.b"] = r(cfg.out_hidden, cfg.hidden * m2), r(cfg.out_hidden)
    return w


@dataclass
class ImageEmbedding:
    rows: torch.Tensor                             # [tokens, out_hidden]
    grid: Tuple[int, int, int]                     # (t, h, w) in TOKENS (after the merge)
    deepstack: List[torch.Tensor] = field(default_factory=list)     # each [tokens, out_hidden]


def _lin(x, w, b=None):
    """x @ w^T (+ b). bf16 rows on a GPU go through the framework's own tensor-core GEMM when the shapes allow
    (K a multiple of 64, N of 8); everything else is a plain tensor operation."""
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 \
            and w.shape[1] % 64 == 0 and w.shape[0] % 8 == 0 and w.is_contiguous():
        from ..ops import sm100
        y = sm100.linear(x.contiguous(), w)
        return y if b is None else y + b
    return F.linear(x, w, b)


def _act(x, kind):
    if kind == "gelu_tanh":
        return F.gelu(x, approximate="tanh")
    if kind == "gelu":
        return F.gelu(x)
    return F.silu(x)


def merge_order_coords(gh: int, gw: int, m: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """(row, column) of every patch in merge order."""
    r = torch.arange(gh, device=device).view(gh // m, m, 1, 1).expand(gh // m, m, gw // m, m)
    c = torch.arange(gw, device=device).view(1, 1, gw // m, m).expand(gh // m, m, gw // m, m)
    return r.permute(0, 2, 1, 3).reshape(-1), c.permute(0, 2, 1, 3).reshape(-1)


class VisionTower:
    def __init__(self, cfg: VisionConfig, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = cfg, weights
        if cfg.hidden % cfg.n_head or (cfg.projector != "pool" and cfg.head_dim % 4):
            raise ValueError("vision tower: hidden must split into heads of a multiple of 4 dims")
        side = int(round(math.sqrt(cfg.num_pos)))
        if side * side != cfg.num_pos:
            raise ValueError("vision tower: the position table must be a square grid")
        self.side = side

    @property
    def device(self):
        return self.w["patch.w"].device

    @property
    def dtype(self):
        return self.w["patch.w"].dtype

    # ------------------------------------------------------------------ pieces
    def _pos_embed(self, gh: int, gw: int, rr: torch.Tensor, cc: torch.Tensor) -> torch.Tensor:
        """Bilinear resampling of the square position table to a gh x gw grid, rows in merge order."""
        n = self.side
        tab = self.w["pos"].float()
        ys = torch.linspace(0, n - 1, gh, device=tab.device)[rr]
        xs = torch.linspace(0, n - 1, gw, device=tab.device)[cc]
        y0, x0 = ys.floor().long(), xs.floor().long()
        y1, x1 = (y0 + 1).clamp(max=n - 1), (x0 + 1).clamp(max=n - 1)
        fy, fx = (ys - y0).unsqueeze(1), (xs - x0).unsqueeze(1)
        out = (tab[y0 * n + x0] * (1 - fy) * (1 - fx) + tab[y0 * n + x1] * (1 - fy) * fx
               + tab[y1 * n + x0] * fy * (1 - fx) + tab[y1 * n + x1] * fy * fx)
        return out

    def _rope(self, rr: torch.Tensor, cc: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """cos / sin [patches, head_dim]: the first quarter of the frequencies turns with the row, the second with
        the column, and the pair repeats for the rotate-half partner dims."""
        hd = self.cfg.head_dim
        q = hd // 4
        inv = 1.0 / (self.cfg.rope_theta ** (torch.arange(0, q, device=rr.device, dtype=torch.float32) / q))
        ang = torch.cat([rr.float()[:, None] * inv[None], cc.float()[:, None] * inv[None]], dim=1)    # [n, hd / 2]
        ang = torch.cat([ang, ang], dim=1)
        return ang.cos(), ang.sin()

    @staticmethod
    def _rotate(x, cos, sin):
        h = x.shape[-1] // 2
        rot = torch.cat([-x[..., h:], x[..., :h]], dim=-1)
        return x * cos[:, None, :] + rot * sin[:, None, :]

    def _merger(self, name: str, x: torch.Tensor, post_shuffle: bool) -> torch.Tensor:
        w, m2 = self.w, self.cfg.spatial_merge_size ** 2
        H = self.cfg.hidden
        if post_shuffle:
            x = F.layer_norm(x.reshape(-1, H * m2), (H * m2,), w[f"{name}.ln.w"], w[f"{name}.ln.b"], self.cfg.ln_eps)
        else:
            x = F.layer_norm(x, (H,), w[f"{name}.ln.w"], w[f"{name}.ln.b"], self.cfg.ln_eps).reshape(-1, H * m2)
        x = F.gelu(_lin(x, w[f"{name}.fc1.w"], w[f"{name}.fc1.b"]))
        return _lin(x, w[f"{name}.fc2.w"], w[f"{name}.fc2.b"])

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def encode(self, patches: torch.Tensor, grid: Tuple[int, int, int]) -> ImageEmbedding:
        cfg, w = self.cfg, self.w
        t, gh, gw = grid
        m = cfg.spatial_merge_size
        if t != 1 or gh % m or gw % m or patches.shape != (gh * gw, cfg.patch_dim):
            raise ValueError(f"vision tower: patches {tuple(patches.shape)} do not match grid {grid}")
        dev, dt = self.device, self.dtype
        x = _lin(patches.to(device=dev, dtype=dt), w["patch.w"], w["patch.b"])
        rr, cc = merge_order_coords(gh, gw, m, dev)
        x = x + self._pos_embed(gh, gw, rr, cc).to(dt)
        use_rope = cfg.projector != "pool"
        if use_rope:
            cos, sin = self._rope(rr, cc)
            cos, sin = cos.to(dt), sin.to(dt)
        n, nh, hd = x.shape[0], cfg.n_head, cfg.head_dim
        deep: List[torch.Tensor] = []
        for i in range(cfg.depth):
            p = f"blk{i}"
            h = F.layer_norm(x, (cfg.hidden,), w[f"{p}.ln1.w"], w[f"{p}.ln1.b"], cfg.ln_eps)
            qkv = _lin(h, w[f"{p}.qkv.w"], w[f"{p}.qkv.b"]).view(n, 3, nh, hd)
            q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
            if use_rope:
                q, k = self._rotate(q, cos, sin), self._rotate(k, cos, sin)
            a = F.scaled_dot_product_attention(q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0),
                                               v.transpose(0, 1).unsqueeze(0))[0].transpose(0, 1).reshape(n, cfg.hidden)
            x = x + _lin(a, w[f"{p}.proj.w"], w[f"{p}.proj.b"])
            h = F.layer_norm(x, (cfg.hidden,), w[f"{p}.ln2.w"], w[f"{p}.ln2.b"], cfg.ln_eps)
            h = _act(_lin(h, w[f"{p}.fc1.w"], w[f"{p}.fc1.b"]), cfg.act)
            x = x + _lin(h, w[f"{p}.fc2.w"], w[f"{p}.fc2.b"])
            if i in cfg.deepstack_layers and cfg.projector != "pool":
                deep.append(self._merger(f"ds{cfg.deepstack_layers.index(i)}", x, True))
        if cfg.projector == "pool":
            pooled = x.view(-1, m * m, cfg.hidden).float().mean(1)
            pooled = pooled * torch.rsqrt(pooled.pow(2).mean(-1, keepdim=True) + cfg.ln_eps) * w["proj.norm.w"].float()
            rows = _lin(pooled.to(dt), w["proj.w"])
        else:
            rows = self._merger("merger", x, False)
        return ImageEmbedding(rows, (1, gh // m, gw // m), deep)
