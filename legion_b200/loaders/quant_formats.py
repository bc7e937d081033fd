"""Block-scaled checkpoint encodings: decode (and encode, for tests and synthetic checkpoints).

NVFP4, ModelOpt layout (``src/hf/nvfp4.rs:5-33`` in the reference): ``weight`` U8 ``[rows, k/2]`` (two
E2M1 codes per byte, low nibble first), ``weight_scale`` F8_E4M3 ``[rows, k/16]``, ``weight_scale_2`` F32
scalar, optional ``input_scale``. compressed-tensors layout: ``weight_packed``, ``weight_scale``,
``weight_global_scale`` where the global scale is a DIVISOR (value = code * block_scale / global_scale).
FP8: ``weight`` F8_E4M3 with ``weight_scale`` (per tensor or per output channel ``[rows, 1]``) or
``weight_scale_inv`` F32 ``[ceil(rows/128), ceil(k/128)]`` (128x128 blocks).
CUDA tensors are decoded by the kernels in ``csrc/quant.cu``; CPU tensors by the torch code below.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def nvfp4_dequant(codes: torch.Tensor, scales: torch.Tensor, global_scale, out_dtype=torch.float32,
                  global_is_divisor: bool = False) -> torch.Tensor:
    """codes U8 [rows, k/2]; scales F8_E4M3 (or U8 bit patterns) [rows, k/16]."""
    gs = float(global_scale) if not torch.is_tensor(global_scale) else float(global_scale.float().reshape(-1)[0])
    if global_is_divisor:
        gs = 1.0 / gs
    if codes.is_cuda:
        from ..ops.sm100 import ext
        out = torch.empty(codes.shape[0], codes.shape[1] * 2, dtype=torch.bfloat16, device=codes.device)
        ext().nvfp4_dequant(codes.contiguous(), scales.view(torch.uint8).contiguous(),
                            torch.tensor([gs], dtype=torch.float32, device=codes.device), out)
        return out.to(out_dtype)
    lut = E2M1_VALUES.to(codes.device)
    lo = lut[(codes & 0xF).long()]
    hi = lut[(codes >> 4).long()]
    vals = torch.stack([lo, hi], dim=-1).reshape(codes.shape[0], -1)
    sc = scales.view(torch.float8_e4m3fn).float() if scales.dtype == torch.uint8 else scales.float()
    vals = vals.view(codes.shape[0], -1, 16) * sc[:, :, None] * gs
    return vals.reshape(codes.shape[0], -1).to(out_dtype)


def nvfp4_quant(w: torch.Tensor, global_scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns (codes U8 [rows, k/2], scales F8_E4M3 [rows, k/16], global scale F32 scalar)."""
    wf = w.float()
    rows, k = wf.shape
    assert k % 16 == 0
    if global_scale is None:
        global_scale = max(float(wf.abs().max()) / (6.0 * 448.0), 1e-12)
    blocks = wf.view(rows, k // 16, 16)
    amax = blocks.abs().amax(-1)
    sc = (amax / 6.0 / global_scale).to(torch.float8_e4m3fn)
    dec = sc.float() * global_scale
    inv = torch.where(dec > 0, 1.0 / dec, torch.zeros_like(dec))
    x = blocks * inv[:, :, None]
    lut = E2M1_VALUES[:8].to(w.device)
    idx = (x.abs()[..., None] - lut).abs().argmin(-1)
    # ties: |x| exactly between two magnitudes picks the even code like round-to-nearest-even
    code = (idx | ((x < 0).long() << 3)).to(torch.uint8).view(rows, k)
    packed = code[:, 0::2] | (code[:, 1::2] << 4)
    return packed.contiguous(), sc, torch.tensor(global_scale, dtype=torch.float32)


def fp8_dequant(w: torch.Tensor, scale: torch.Tensor, block: Optional[Tuple[int, int]] = None,
                out_dtype=torch.float32) -> torch.Tensor:
    """w F8_E4M3 [rows, k]; scale: scalar, [rows] / [rows, 1], or block grid when ``block`` is given."""
    if block is not None:
        br, bk = block
        if w.is_cuda:
            from ..ops.sm100 import ext
            out = torch.empty(w.shape, dtype=torch.bfloat16, device=w.device)
            ext().fp8_block_dequant(w.view(torch.uint8).contiguous(), scale.float().contiguous(), br, bk, out)
            return out.to(out_dtype)
        rows, k = w.shape
        s = scale.float().repeat_interleave(br, 0)[:rows].repeat_interleave(bk, 1)[:, :k]
        return (w.float() * s).to(out_dtype)
    s = scale.float()
    if s.numel() == 1:
        return (w.float() * s.reshape(())).to(out_dtype)
    return (w.float() * s.reshape(-1, 1)).to(out_dtype)


def fp8_block_quant(w: torch.Tensor, block=(128, 128)) -> Tuple[torch.Tensor, torch.Tensor]:
    br, bk = block
    rows, k = w.shape
    R, K = (rows + br - 1) // br, (k + bk - 1) // bk
    pad = torch.zeros(R * br, K * bk, dtype=torch.float32, device=w.device)
    pad[:rows, :k] = w.float()
    blocks = pad.view(R, br, K, bk)
    amax = blocks.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    q = (blocks / scale[:, None, :, None]).view(R * br, K * bk)[:rows, :k].to(torch.float8_e4m3fn)
    return q, scale


def fp8_act_quant(x: torch.Tensor, group: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token, per-``group``-channel activation scales (1 x 128): returns (F8_E4M3 codes, scales)."""
    T, k = x.shape
    g = x.float().view(T, k // group, group)
    amax = g.abs().amax(-1)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    return (g / scale[:, :, None]).view(T, k).to(torch.float8_e4m3fn), scale
