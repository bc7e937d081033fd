"""Image decoding and preprocessing for the vision towers.

An image is decoded to RGB (PNG, JPEG, WebP, GIF: the formats the API accepts), resized so that both sides are
multiples of ``patch_size * spatial_merge_size`` and the area lies within the tower's pixel budget, normalised with
the tower's mean / std, and cut into patches. Patches leave in "merge order": the ``merge x merge`` patches that
become one language-model token are consecutive, blocks in row-major order, which is the order the Qwen3-VL merger
and the pooling projector consume.

Two resize policies, as in the reference (``src/vision/mod.rs:46-48``, ``src/vision/preprocess.rs``): ``pad`` keeps
the aspect ratio and centres the image on a black canvas of the aligned size (Qwen3-VL mmproj files), ``stretch``
resizes to the aligned size itself (Gemma 4)."""
from __future__ import annotations

import io
import math
from dataclasses import dataclass, field
from typing import Tuple

import torch


class VisionError(ValueError):
    pass


@dataclass
class VisionHparams:
    patch_size: int = 16
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    image_min_pixels: int = 0          # 0 = 8 tokens' worth
    image_max_pixels: int = 0          # 0 = 4096 tokens' worth
    image_mean: Tuple[float, float, float] = (0.5, 0.5, 0.5)
    image_std: Tuple[float, float, float] = (0.5, 0.5, 0.5)
    resize: str = "pad"                # "pad" | "stretch"
    min_tokens: int = 8
    max_tokens: int = 4096

    def __post_init__(self):
        f = self.patch_size * self.spatial_merge_size
        if self.patch_size <= 0 or self.spatial_merge_size <= 0 or f > 65536:
            raise VisionError("patch / merge size out of range")
        if not self.image_min_pixels:
            self.image_min_pixels = f * f * self.min_tokens
        if not self.image_max_pixels:
            self.image_max_pixels = f * f * self.max_tokens
        if self.image_max_pixels < self.image_min_pixels:
            raise VisionError("image_max_pixels < image_min_pixels")
        if any(s <= 0 or not math.isfinite(s) for s in self.image_std):
            raise VisionError("image_std must be positive")

    @property
    def factor(self) -> int:
        return self.patch_size * self.spatial_merge_size

    def max_image_tokens(self) -> int:
        return self.image_max_pixels // (self.factor * self.factor)


@dataclass
class Preprocessed:
    patches: torch.Tensor              # [n_patches, 3 * temporal * patch * patch] float32, merge order
    grid: Tuple[int, int, int]         # (t, h, w) in patches
    size: Tuple[int, int] = field(default=(0, 0))      # pixels (height, width) after the resize

    @property
    def n_patches(self) -> int:
        return self.grid[0] * self.grid[1] * self.grid[2]


def decode_image(data: bytes) -> torch.Tensor:
    """Encoded image bytes -> uint8 [H, W, 3] RGB (first frame of an animation; alpha composited on white)."""
    try:
        from PIL import Image
    except ImportError as e:              # pragma: no cover - PIL ships with the image
        raise VisionError("image decoding needs Pillow") from e
    try:
        im = Image.open(io.BytesIO(data))
        im.load()
    except Exception as e:
        raise VisionError(f"invalid or unsupported image: {e}") from None
    if im.mode in ("RGBA", "LA") or (im.mode == "P" and "transparency" in im.info):
        rgba = im.convert("RGBA")
        bg = Image.new("RGBA", rgba.size, (255, 255, 255, 255))
        im = Image.alpha_composite(bg, rgba).convert("RGB")
    else:
        im = im.convert("RGB")
    w, h = im.size
    if w <= 0 or h <= 0 or w * h > (1 << 28):
        raise VisionError("image dimensions are out of range")
    return torch.frombuffer(bytearray(im.tobytes()), dtype=torch.uint8).view(h, w, 3)


def smart_size(height: int, width: int, factor: int, min_pixels: int, max_pixels: int) -> Tuple[int, int]:
    """Target (height, width): multiples of ``factor`` close to the original, scaled into the pixel budget with the
    aspect ratio kept."""
    if height <= 0 or width <= 0:
        raise VisionError("image dimensions are out of range")
    if max(height, width) / min(height, width) > 200:
        raise VisionError("aspect ratio above 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def _resize(img: torch.Tensor, h: int, w: int) -> torch.Tensor:
    """uint8 [H, W, 3] -> float32 [3, h, w] in 0..1, bicubic with antialiasing."""
    x = img.permute(2, 0, 1).unsqueeze(0).float() / 255.0
    if x.shape[-2:] != (h, w):
        x = torch.nn.functional.interpolate(x, size=(h, w), mode="bicubic", align_corners=False, antialias=True)
    return x[0].clamp_(0.0, 1.0)


def preprocess(img: torch.Tensor, hp: VisionHparams) -> Preprocessed:
    """uint8 [H, W, 3] -> normalised patches in merge order."""
    H, W = int(img.shape[0]), int(img.shape[1])
    th, tw = smart_size(H, W, hp.factor, hp.image_min_pixels, hp.image_max_pixels)
    if hp.resize == "stretch":
        x = _resize(img, th, tw)
    else:
        # aspect kept: scale to fit inside the aligned canvas, centre on black
        s = min(th / H, tw / W)
        ih, iw = max(1, min(th, round(H * s))), max(1, min(tw, round(W * s)))
        inner = _resize(img, ih, iw)
        x = torch.zeros(3, th, tw)
        y0, x0 = (th - ih) // 2, (tw - iw) // 2
        x[:, y0:y0 + ih, x0:x0 + iw] = inner
    mean = torch.tensor(hp.image_mean).view(3, 1, 1)
    std = torch.tensor(hp.image_std).view(3, 1, 1)
    x = (x - mean) / std
    P, m, tp = hp.patch_size, hp.spatial_merge_size, hp.temporal_patch_size
    gh, gw = th // P, tw // P
    # a still image is its own second frame: [tp, 3, th, tw]
    frames = x.unsqueeze(0).expand(tp, -1, -1, -1)
    # [tp, 3, gh/m, m, P, gw/m, m, P] -> [gh/m, gw/m, m, m, 3, tp, P, P]
    v = frames.reshape(tp, 3, gh // m, m, P, gw // m, m, P).permute(2, 5, 3, 6, 1, 0, 4, 7)
    patches = v.reshape(gh * gw, 3 * tp * P * P).contiguous()
    return Preprocessed(patches, (1, gh, gw), (th, tw))
