"""The Gemma 4 vision tower: one image's patches to rows of the language model's width, one row per k x k block of
patches (k = ``pooling_kernel_size``).

1. Patches: pixels in [0, 1] scaled to [-1, 1], one linear map per patch (no bias), plus two learned position rows,
   one looked up by the patch's column and one by its row.
2. Blocks: RMS-normed ViT blocks with separate q / k / v; q and k RMS-normed per head with weights, v without;
   rotary embedding in two halves of each head (first half turns with the column, second half with the row, base
   100); full attention at scale 1; the attention output and the GELU-gated MLP output are RMS-normed before they
   join the residual.
3. Pooler: each k x k block of patches averaged, scaled by sqrt(width), optionally standardised
   (``(x - std_bias) * std_scale``), RMS-normed without a weight and projected to the language model's width.

Patches arrive in merge order (the k x k blocks contiguous, ``vision.preprocess`` with ``spatial_merge_size = k`` and
``temporal_patch_size = 1``, channel-major inside a patch); attention does not depend on the order and pooling then is
a mean over consecutive rows. Reference counterpart: ``src/vision/gemma4v.rs`` (which follows llama.cpp's
``gemma4v`` graph); the Hugging Face ``Gemma4VisionModel`` + ``Gemma4MultimodalEmbedder`` compute the same thing and
are what the parity test compares with. Towers with clipped linears (``use_clipped_linears``) are refused, as the
reference refuses them."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Tuple

import torch
import torch.nn.functional as F

from .tower import ImageEmbedding, _act, _lin, merge_order_coords


@dataclass
class Gemma4VisionConfig:
    depth: int = 2
    hidden: int = 32
    n_head: int = 2
    n_kv_head: int = 2
    head_dim: int = 16
    intermediate: int = 64
    out_hidden: int = 64               # width of the language model
    patch_size: int = 16
    spatial_merge_size: int = 3        # the pooling kernel: k x k patches become one row
    temporal_patch_size: int = 1
    num_pos: int = 64                  # rows of each of the two position tables
    act: str = "gelu_tanh"
    ln_eps: float = 1e-6
    rope_theta: float = 100.0
    standardize: bool = False
    deepstack_layers: Tuple[int, ...] = ()
    projector: str = "gemma4v"

    @property
    def patch_dim(self) -> int:
        return 3 * self.patch_size * self.patch_size


def random_gemma4v_weights(cfg: Gemma4VisionConfig, device="cpu", dtype=torch.float32, seed: int = 0, std: float = 0.05):
    g = torch.Generator().manual_seed(seed)
    r = lambda *shape: (torch.randn(*shape, generator=g) * std).to(device=device, dtype=dtype)       # noqa: E731
    one = lambda n: (1.0 + 0.1 * torch.randn(n, generator=g)).to(device=device, dtype=dtype)          # noqa: E731
    H, D = cfg.hidden, cfg.head_dim
    w = {"patch.w": r(H, cfg.patch_dim), "pos.x": r(cfg.num_pos, H), "pos.y": r(cfg.num_pos, H),
         "proj.w": r(cfg.out_hidden, H)}
    if cfg.standardize:
        w["std.bias"], w["std.scale"] = r(H), one(H)
    for i in range(cfg.depth):
        p = f"blk{i}"
        w.update({f"{p}.q.w": r(cfg.n_head * D, H), f"{p}.k.w": r(cfg.n_kv_head * D, H), f"{p}.v.w": r(cfg.n_kv_head * D, H),
                  f"{p}.o.w": r(H, cfg.n_head * D), f"{p}.q_norm.w": one(D), f"{p}.k_norm.w": one(D),
                  f"{p}.ln1.w": one(H), f"{p}.post_attn.w": one(H), f"{p}.ln2.w": one(H), f"{p}.post_ffn.w": one(H),
                  f"{p}.gate.w": r(cfg.intermediate, H), f"{p}.up.w": r(cfg.intermediate, H),
                  f"{p}.down.w": r(H, cfg.intermediate)})
    return w


def _rms(x: torch.Tensor, eps: float, w=None) -> torch.Tensor:
    y = x.float()
    y = y * torch.pow(y.pow(2).mean(-1, keepdim=True) + eps, -0.5)
    if w is not None:
        y = y * w.float()
    return y.to(x.dtype)


class Gemma4VisionTower:
    def __init__(self, cfg: Gemma4VisionConfig, weights: Dict[str, torch.Tensor]):
        if cfg.head_dim % 4:
            raise ValueError("gemma4v: the head size must divide by 4 (two rotary halves of frequency pairs)")
        self.cfg, self.w = cfg, weights

    @property
    def device(self):
        return self.w["patch.w"].device

    @property
    def dtype(self):
        return self.w["patch.w"].dtype

    def _rope(self, rr: torch.Tensor, cc: torch.Tensor):
        """cos / sin [n, head_dim]: the first half of a head turns with the column, the second with the row; inside
        a half the pairs are (i, i + quarter)."""
        half = self.cfg.head_dim // 2
        inv = 1.0 / (self.cfg.rope_theta ** (torch.arange(0, half, 2, device=rr.device, dtype=torch.float32) / half))
        parts = []
        for pos in (cc, rr):
            f = pos.float()[:, None] * inv[None]
            parts.append(torch.cat([f, f], dim=-1))
        ang = torch.cat(parts, dim=-1)
        return ang.cos(), ang.sin()

    @staticmethod
    def _rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """x [n, heads, D]; each half of D is rotated on its own."""
        half = x.shape[-1] // 2
        q = half // 2
        out = []
        for h in range(2):
            t = x[..., h * half:(h + 1) * half]
            rot = torch.cat([-t[..., q:], t[..., :q]], dim=-1)
            c, s = cos[:, None, h * half:(h + 1) * half], sin[:, None, h * half:(h + 1) * half]
            out.append(t * c + rot * s)
        return torch.cat(out, dim=-1)

    def encode(self, patches: torch.Tensor, grid: Tuple[int, int, int]) -> ImageEmbedding:
        cfg, w = self.cfg, self.w
        t, gh, gw = grid
        k = cfg.spatial_merge_size
        if t != 1 or gh % k or gw % k or patches.shape != (gh * gw, cfg.patch_dim):
            raise ValueError(f"gemma4v tower: patches {tuple(patches.shape)} do not match grid {grid}")
        if max(gh, gw) > cfg.num_pos:
            raise ValueError(f"gemma4v tower: a {gh} x {gw} patch grid exceeds the {cfg.num_pos} learned positions")
        dev, dt = self.device, self.dtype
        rr, cc = merge_order_coords(gh, gw, k, dev)
        x = _lin((2.0 * (patches.to(device=dev, dtype=torch.float32) - 0.5)).to(dt), w["patch.w"])
        x = x + w["pos.x"][cc] + w["pos.y"][rr]
        cos, sin = self._rope(rr, cc)
        cos, sin = cos.to(dt), sin.to(dt)
        n, nh, nkv, D = x.shape[0], cfg.n_head, cfg.n_kv_head, cfg.head_dim
        for i in range(cfg.depth):
            p = f"blk{i}"
            h = _rms(x, cfg.ln_eps, w[f"{p}.ln1.w"])
            q = _rms(_lin(h, w[f"{p}.q.w"]).view(n, nh, D), cfg.ln_eps, w[f"{p}.q_norm.w"])
            kk = _rms(_lin(h, w[f"{p}.k.w"]).view(n, nkv, D), cfg.ln_eps, w[f"{p}.k_norm.w"])
            v = _rms(_lin(h, w[f"{p}.v.w"]).view(n, nkv, D), cfg.ln_eps)
            q, kk = self._rotate(q, cos, sin), self._rotate(kk, cos, sin)
            if nkv != nh:
                kk, v = kk.repeat_interleave(nh // nkv, dim=1), v.repeat_interleave(nh // nkv, dim=1)
            a = F.scaled_dot_product_attention(q.transpose(0, 1).unsqueeze(0), kk.transpose(0, 1).unsqueeze(0),
                                               v.transpose(0, 1).unsqueeze(0), scale=1.0)[0]
            a = _lin(a.transpose(0, 1).reshape(n, nh * D), w[f"{p}.o.w"])
            x = x + _rms(a, cfg.ln_eps, w[f"{p}.post_attn.w"])
            h = _rms(x, cfg.ln_eps, w[f"{p}.ln2.w"])
            h = _lin(_act(_lin(h, w[f"{p}.gate.w"]), cfg.act) * _lin(h, w[f"{p}.up.w"]), w[f"{p}.down.w"])
            x = x + _rms(h, cfg.ln_eps, w[f"{p}.post_ffn.w"])
        pooled = x.view(-1, k * k, cfg.hidden).float().mean(1) * cfg.hidden ** 0.5
        if cfg.standardize:
            pooled = (pooled - w["std.bias"].float()) * w["std.scale"].float()
        rows = _lin(_rms(pooled, cfg.ln_eps).to(dt), w["proj.w"])
        return ImageEmbedding(rows, (1, gh // k, gw // k), [])
