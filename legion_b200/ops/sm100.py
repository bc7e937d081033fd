"""Python front-ends of the sm_100a kernels in ``legion_b200/_C.so``.

Every function takes CUDA tensors, enqueues on the current stream and never synchronises; scratch
(split-K partials, attention split buffers, routing plans) comes from a per-device ``Workspace`` that
is allocated once, so a decode step captured in a CUDA graph replays without allocator traffic.
The extension is required on a GPU: there is no silent fallback to eager PyTorch.
"""
from __future__ import annotations

import importlib
import os
import threading
from typing import Optional

import torch

_C = None
_C_err: Optional[BaseException] = None
_lock = threading.Lock()


# kernels launched by one call of each binding (for the launch counter)
KERNELS_PER_CALL = {"moe_plan": 3, "paged_decode": 1, "argmax": 2, "wgemm_workspace_floats": 0}
LAUNCHES = {"n": 0}


class _Counting:
    """Proxy of the extension module that counts kernel launches (``LAUNCHES['n']``) and, with ``LB_OP_PROFILE=1``
    (or ``op_profile(True)``), times every op between two CUDA events: the per-op table of the reference's
    ``LEGION_OP_PROFILE`` (``src/ggml/op_profile.rs:1-16``). Profiling is for eager steps (run with
    ``--no-cuda-graphs``); captured graphs replay without passing through here."""

    def __init__(self, mod):
        self._mod = mod
        self._cache = {}

    def __getattr__(self, name):
        f = self._cache.get(name)
        if f is None:
            raw = getattr(self._mod, name)
            k = KERNELS_PER_CALL.get(name, 1)

            def f(*a, _raw=raw, _k=k, _name=name, **kw):
                LAUNCHES["n"] += _k
                if not OP_PROFILE["on"] or _k == 0 or torch.cuda.is_current_stream_capturing():
                    return _raw(*a, **kw)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                out = _raw(*a, **kw)
                e1.record()
                OP_PROFILE["events"].append((_name, e0, e1))
                return out
            self._cache[name] = f
        return f


OP_PROFILE = {"on": os.environ.get("LB_OP_PROFILE", "0") == "1", "events": []}


def op_profile(on: bool):
    OP_PROFILE["on"] = bool(on)
    OP_PROFILE["events"].clear()


def op_profile_report(reset: bool = True):
    """Rows (op, calls, total ms, mean us, share) of the ops timed since the last report, slowest first."""
    torch.cuda.synchronize()
    agg = {}
    for name, e0, e1 in OP_PROFILE["events"]:
        c = agg.setdefault(name, [0, 0.0])
        c[0] += 1
        c[1] += e0.elapsed_time(e1)
    if reset:
        OP_PROFILE["events"].clear()
    total = sum(v[1] for v in agg.values()) or 1.0
    return [(n, c, ms, ms / c * 1e3, ms / total) for n, (c, ms) in sorted(agg.items(), key=lambda kv: -kv[1][1])]


def ext():
    """Returns the extension module, importing ``legion_b200._C`` on first use."""
    global _C, _C_err
    if _C is None and _C_err is None:
        with _lock:
            if _C is None and _C_err is None:
                try:
                    mod = importlib.import_module("legion_b200._C")
                    mod.set_pdl(bool(TUNE["pdl"]))
                    _C = _Counting(mod)
                except BaseException as e:  # missing .so, ABI mismatch, missing libcudart
                    _C_err = e
    if _C is None:
        raise RuntimeError(
            "legion_b200._C (the sm_100a extension) is not importable: build it with "
            "`python -m legion_b200.build_ext`") from _C_err
    return _C


def have_ext() -> bool:
    try:
        ext()
        return True
    except RuntimeError:
        return False


NUM_SMS = 148

# tuning knobs (environment: LB_TUNE="decode_fixed_tiles=2,dense_route=1")
TUNE = {"decode_lanes": 2, "nv4_sorted": 1, "fp8_fused_quant": 1, "nv4_sorted_bn": 64, "gdn_chunk": 1, "decode_fixed_tiles": 2, "fused_plan": 1, "fused_router": 1, "dense_route": 1, "pdl": 1, "route_norm": 0, "mla_head_gemm": 1}
for _kv in os.environ.get("LB_TUNE", "").split(","):
    if "=" in _kv:
        TUNE[_kv.split("=")[0].strip()] = int(_kv.split("=")[1])


_CANARY_ON = os.environ.get("LB_CANARY", "0") == "1"


class Workspace:
    """Per-device scratch shared by all kernels on that device's compute stream. A decode step that runs as several
    concurrent lanes (``engine.cuda_graphs``: independent halves of the batch on parallel branches of one CUDA graph)
    gives every lane a workspace of its own: ``Workspace.lane`` selects it while that lane's launches are issued."""

    _by_device: dict = {}
    lane: int = 0

    def __init__(self, device: torch.device):
        self.device = device
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.counters = torch.zeros(1 << 16, dtype=torch.int32, device=device)
        self.splitk = torch.empty(1 << 23, dtype=torch.float32, device=device)  # 32 MiB
        self._attn: dict = {}
        self._cache: dict = {}
        self._guards: dict = {}

    @classmethod
    def get(cls, device) -> "Workspace":
        device = torch.device(device)
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        key = device if cls.lane == 0 else (device, cls.lane)
        ws = cls._by_device.get(key)
        if ws is None:
            ws = cls(device)
            cls._by_device[key] = ws
        return ws

    CANARY_BYTES = 256
    CANARY = 0xA5

    def buf(self, key, shape, dtype):
        """A cached scratch tensor: same key and size -> same storage (graph-safe). With ``LB_CANARY=1`` every buffer
        sits between two guard areas filled with a byte pattern that ``check_canaries`` verifies: the substitute
        for a memory checker on kernels that index scratch memory (a write past either end shows up by name)."""
        k = (key, tuple(shape), dtype)
        t = self._cache.get(k)
        if t is None:
            if _CANARY_ON:
                n = 1
                for d in shape:
                    n *= int(d)
                nbytes = n * torch.empty(0, dtype=dtype).element_size()
                pad = self.CANARY_BYTES
                raw = torch.full((nbytes + 2 * pad,), self.CANARY, dtype=torch.uint8, device=self.device)
                t = raw[pad:pad + nbytes].view(dtype).view(shape)
                self._guards[k] = raw
            else:
                t = torch.empty(shape, dtype=dtype, device=self.device)
            self._cache[k] = t
        return t

    def check_canaries(self) -> list:
        """Names of the scratch buffers whose guard areas no longer hold the pattern (``LB_CANARY=1`` only)."""
        bad = []
        pad = self.CANARY_BYTES
        for k, raw in self._guards.items():
            if bool((raw[:pad] != self.CANARY).any()) or bool((raw[-pad:] != self.CANARY).any()):
                bad.append(str(k[0]))
        return bad

    def check(self) -> int:
        """Synchronises and returns the kernels' status word (0 = ok); clears it."""
        v = int(self.status[0].item())
        if v:
            self.status.zero_()
        for key, other in list(self._by_device.items()):      # the other lanes of this device
            if isinstance(key, tuple) and key[0] == self.device and other is not self:
                ov = int(other.status[0].item())
                if ov:
                    other.status.zero_()
                    v = v or ov
        return v


class QWeight:
    """NVFP4 weight kept in its 4-bit encoding: ``codes`` uint8 [..., rows, K/2] (two e2m1 values per byte, low
    nibble first), ``scales`` uint8 e4m3 bit patterns [..., rows, K/16], ``gscale`` float32 per tensor (per expert;
    for a fused gate/up tensor two values per expert: gate, up). The GEMM streams the 4-bit bytes and expands
    them to bf16 operand tiles inside the kernel (``csrc/gemm_sm100.cu``), so a decode step reads 0.56 bytes per
    weight instead of 2."""
    __slots__ = ("codes", "scales", "gscale")

    def __init__(self, codes, scales, gscale):
        self.codes, self.scales, self.gscale = codes, scales.view(torch.uint8), gscale.float().reshape(-1).contiguous()

    @property
    def shape(self):
        return tuple(self.codes.shape[:-1]) + (self.codes.shape[-1] * 2,)

    @property
    def device(self):
        return self.codes.device

    def dim(self):
        return self.codes.dim()

    def view2d(self):
        return self.codes.reshape(-1, self.codes.shape[-1]), self.scales.reshape(-1, self.scales.shape[-1])

    def narrow(self, lo: int, hi: int) -> "QWeight":
        """Groups [lo, hi) of a stacked weight (a view: no copy). hi == lo + 1 with ``squeeze`` semantics is
        ``narrow(lo, lo + 1).squeeze0()``."""
        per = self.gscale.numel() // self.codes.shape[0]
        return QWeight(self.codes[lo:hi], self.scales[lo:hi], self.gscale[lo * per:hi * per])

    def squeeze0(self) -> "QWeight":
        return QWeight(self.codes[0], self.scales[0], self.gscale)

    @classmethod
    def quantize(cls, w: torch.Tensor, dual_rows: int = 0):
        """Encodes a bf16/fp32 weight [..., rows, K] (tests, synthetic checkpoints). ``dual_rows`` > 0: the tensor is
        a fused [gate | up] stack of 2 * dual_rows rows and each half gets its own tensor scale."""
        from ..loaders.quant_formats import nvfp4_quant
        lead = w.shape[:-2]
        flat = w.reshape(-1, w.shape[-2], w.shape[-1])
        codes, scales, gs = [], [], []
        for t in flat:
            parts = [t] if not dual_rows else [t[:dual_rows], t[dual_rows:]]
            cs, ss = [], []
            for part in parts:
                c, sc, g = nvfp4_quant(part.float().cpu())
                cs.append(c)
                ss.append(sc.view(torch.uint8))
                gs.append(float(g))
            codes.append(torch.cat(cs, 0))
            scales.append(torch.cat(ss, 0))
        dev = w.device
        return cls(torch.stack(codes).reshape(*lead, *codes[0].shape).to(dev),
                   torch.stack(scales).reshape(*lead, *scales[0].shape).to(dev),
                   torch.tensor(gs, dtype=torch.float32, device=dev))

    @classmethod
    def quantize_cuda(cls, w: torch.Tensor, dual_rows: int = 0):
        """Device-side encoding of a CUDA bf16 weight [..., rows, K] (``csrc/quant.cu::nvfp4_quant``): one tensor
        scale per leading index (two with ``dual_rows``: gate rows, up rows)."""
        C = ext()
        rows, K = w.shape[-2], w.shape[-1]
        flat = w.reshape(-1, rows, K)
        n = flat.shape[0]
        codes = torch.empty(n, rows, K // 2, dtype=torch.uint8, device=w.device)
        scales = torch.empty(n, rows, K // 16, dtype=torch.uint8, device=w.device)
        per = 2 if dual_rows else 1
        gs = torch.empty(n * per, dtype=torch.float32, device=w.device)
        for t in range(n):
            for h in range(per):
                r0, r1 = (0, rows) if not dual_rows else (h * dual_rows, (h + 1) * dual_rows)
                part = flat[t, r0:r1]
                g = (part.float().abs().max() / (6.0 * 448.0)).clamp_min(1e-12).reshape(1)
                gs[t * per + h] = g[0]
                C.nvfp4_quant(part.contiguous(), g, codes[t, r0:r1], scales[t, r0:r1])
        lead = tuple(w.shape[:-2])
        return cls(codes.reshape(*lead, rows, K // 2), scales.reshape(*lead, rows, K // 16), gs)

    def dequantize(self, dtype=torch.bfloat16):
        from ..loaders.quant_formats import nvfp4_dequant
        c2, s2 = self.view2d()
        rows = self.codes.shape[-2]
        n_t = c2.shape[0] // rows
        per = self.gscale.numel() // n_t
        out = torch.empty(c2.shape[0], c2.shape[1] * 2, dtype=dtype, device=self.device)
        for t in range(n_t):
            for h in range(per):
                r0 = t * rows + h * (rows // per)
                r1 = r0 + rows // per
                out[r0:r1] = nvfp4_dequant(c2[r0:r1].cpu(), s2[r0:r1].cpu(), float(self.gscale[t * per + h]),
                                           out_dtype=dtype).to(self.device)
        return out.reshape(self.shape)


class Nv4Weight:
    """NVFP4 weight in the layout of the native block-scaled GEMM (``csrc/gemm_nvfp4_sm100.cu``): ``codes`` uint8
    [..., rows, K/2] exactly as shipped (two e2m1 values per byte, low nibble first), ``sf`` the UE4M3 block scales
    re-ordered into 512-byte atoms (128 rows x 4 blocks, the order tcgen05.cp wants; same bytes, other order),
    ``gscale`` float32 per tensor (per expert; two per expert for a fused gate/up stack). Rows per leading index
    must be a multiple of 128. Activations are quantised to NVFP4 as well (W4A4), so the tensor cores run the
    e2m1 x e2m1 block-scaled instruction and nothing is expanded."""
    __slots__ = ("codes", "sf", "gscale", "scales_lin")

    def __init__(self, codes, sf, gscale, scales_lin=None):
        self.codes, self.sf, self.gscale = codes, sf, gscale.float().reshape(-1).contiguous()
        self.scales_lin = scales_lin          # kept only when asked for (tests / de-quantisation)

    @property
    def shape(self):
        return tuple(self.codes.shape[:-1]) + (self.codes.shape[-1] * 2,)

    @property
    def device(self):
        return self.codes.device

    def dim(self):
        return self.codes.dim()

    def view2d(self):
        return self.codes.reshape(-1, self.codes.shape[-1])

    @classmethod
    def from_parts(cls, codes, scales, gscale, keep_linear: bool = False):
        """From the checkpoint tensors: codes [..., rows, K/2], scales e4m3 bytes [..., rows, K/16], tensor scale(s)."""
        C = ext()
        rows = codes.shape[-2]
        if codes.dim() > 2 and rows % 128:
            raise ValueError("stacked NVFP4 weights need a multiple of 128 rows per slice")
        c2 = codes.reshape(-1, codes.shape[-1]).contiguous()
        s2 = scales.view(torch.uint8).reshape(-1, scales.shape[-1]).contiguous()
        K = c2.shape[1] * 2
        atoms = torch.zeros(C.nv4_sf_bytes(c2.shape[0], K), dtype=torch.uint8, device=codes.device)
        C.nv4_pack_scales(s2, atoms)
        return cls(codes.contiguous(), atoms, gscale, s2 if keep_linear else None)

    @classmethod
    def from_qweight(cls, q: "QWeight", keep_linear: bool = False):
        return cls.from_parts(q.codes, q.scales, q.gscale, keep_linear)

    @classmethod
    def quantize_cuda(cls, w: torch.Tensor, dual_rows: int = 0, keep_linear: bool = False):
        return cls.from_qweight(QWeight.quantize_cuda(w, dual_rows), keep_linear)

    def narrow(self, lo: int, hi: int) -> "Nv4Weight":
        """Groups [lo, hi) of a stacked weight (views of the same storage)."""
        n, rows = self.codes.shape[0], self.codes.shape[-2]
        per = self.gscale.numel() // n
        bpg = self.sf.numel() // n                    # scale-atom bytes per group (rows are a multiple of 128)
        lin = None
        if self.scales_lin is not None:
            lin = self.scales_lin[lo * rows:hi * rows]
        return Nv4Weight(self.codes[lo:hi], self.sf[lo * bpg:hi * bpg], self.gscale[lo * per:hi * per], lin)

    def squeeze0(self) -> "Nv4Weight":
        return Nv4Weight(self.codes[0], self.sf, self.gscale, self.scales_lin)

    def as_qweight(self) -> "QWeight":
        """The same weight with its block scales in the checkpoint's linear order (for the de-quantising GEMM that
        serves prompt-sized steps); the linear copy is made on first use and kept."""
        if self.scales_lin is None:
            C = ext()
            c2 = self.view2d()
            K = c2.shape[1] * 2
            lin = torch.empty(c2.shape[0], K // 16, dtype=torch.uint8, device=self.device)
            C.nv4_unpack_scales(self.sf, lin)
            self.scales_lin = lin
        K16 = self.codes.shape[-1] // 8
        return QWeight(self.codes, self.scales_lin.view(*self.codes.shape[:-1], K16), self.gscale)

    def dequantize(self, dtype=torch.bfloat16):
        return self.as_qweight().dequantize(dtype)


class Nv4Act:
    """NVFP4-encoded activation rows: codes [T, K/2], scale atoms, and the fp32 scale (one per row, or one device
    scalar for all rows when ``stride`` is 0)."""
    __slots__ = ("codes", "sf", "gscale", "stride", "normed", "summed")

    def __init__(self, codes, sf, gscale, stride, normed=None, summed=None):
        self.codes, self.sf, self.gscale, self.stride, self.normed, self.summed = codes, sf, gscale, stride, normed, summed

    def dequantize(self):
        C = ext()
        T, K = self.codes.shape[0], self.codes.shape[1] * 2
        lin = torch.empty(T, K // 16, dtype=torch.uint8, device=self.codes.device)
        C.nv4_unpack_scales(self.sf, lin)
        from ..loaders.quant_formats import nvfp4_dequant
        out = nvfp4_dequant(self.codes.cpu(), lin.cpu(), 1.0, out_dtype=torch.float32).to(self.codes.device)
        g = self.gscale.reshape(-1)[:1] if self.stride == 0 else self.gscale[:T]
        return out * g.reshape(-1, 1)


def nv4_quant_act(x, norm=None, residual=None, static_scale=None, want_normed: bool = False, key=None):
    """bf16 rows [T, K] -> ``Nv4Act``. ``norm=(weight, eps, w_offset)`` fuses the RMSNorm that produces the rows
    (and ``residual`` the add before it: ``summed`` is then the new residual stream); ``static_scale`` is a device
    scalar used for every row instead of the per-row amax scale. ``key``: reuse the same output storage on every
    call with that key (graph-safe)."""
    C = ext()
    T, K = x.shape
    ws = Workspace.get(x.device)
    if key is not None:
        codes = ws.buf((key, "c"), (T, K // 2), torch.uint8)
        sf = ws.buf((key, "s"), (C.nv4_sf_bytes(T, K),), torch.uint8)
        gs = ws.buf((key, "g"), (max(T, 1),), torch.float32) if static_scale is None else static_scale
    else:
        codes = torch.empty(T, K // 2, dtype=torch.uint8, device=x.device)
        sf = torch.empty(C.nv4_sf_bytes(T, K), dtype=torch.uint8, device=x.device)
        gs = torch.empty(max(T, 1), dtype=torch.float32, device=x.device) if static_scale is None else static_scale
    normed = torch.empty_like(x) if (want_normed and norm is not None) else None
    summed = torch.empty_like(x) if residual is not None else None
    C.nv4_act_quant(x, residual, summed, norm[0] if norm else None, norm[1] if norm else 0.0, norm[2] if norm else 0.0,
                    normed, static_scale, codes, sf, None if static_scale is not None else gs)
    return Nv4Act(codes, sf, gs, 0 if static_scale is not None else 1, normed, summed)


def linear_nv4(xq: "Nv4Act", w: "Nv4Weight", residual=None, out=None, bn=None):
    """out[T, N] = dequant(xq) @ dequant(w)^T (+ residual) on the native NVFP4 tensor-core path."""
    C = ext()
    T = xq.codes.shape[0]
    N = w.shape[0]
    if out is None:
        out = torch.empty(T, N, dtype=torch.bfloat16, device=xq.codes.device)
    if T == 0:
        return out
    ws = Workspace.get(xq.codes.device)
    bn = bn or (32 if T <= 32 else (64 if T <= 64 else 128))
    C.wgemm_nv4(w.view2d(), w.sf, w.gscale, xq.codes, xq.sf, xq.gscale, xq.stride, out, residual, None, None, N, False,
                0, 0, bn, ws.status, None, None, None, None, 0, 0, T, None, None, None, None)
    return out


def gate_up_nv4(xq: "Nv4Act", w: "Nv4Weight", n_ff: int, act: str = "silu", out=None, q_scale=None, bn=None):
    """act(x Wg^T) * (x Wu^T) with Wg = w[:n_ff], Wu = w[n_ff:]. With ``q_scale`` (device scalar) the result is
    returned NVFP4-encoded (``Nv4Act`` with that static tensor scale) for the next GEMM."""
    C = ext()
    T = xq.codes.shape[0]
    dev = xq.codes.device
    ws = Workspace.get(dev)
    bn = bn or (32 if T <= 32 else 64)
    a = 0 if act == "silu" else 1
    if q_scale is not None:
        qc = torch.empty(T, n_ff // 2, dtype=torch.uint8, device=dev)
        qs = torch.zeros(C.nv4_sf_bytes(T, n_ff), dtype=torch.uint8, device=dev)
        C.wgemm_nv4(w.view2d(), w.sf, w.gscale, xq.codes, xq.sf, xq.gscale, xq.stride, None, None, None, None, n_ff,
                    True, n_ff, a, bn, ws.status, None, None, None, None, 0, 0, T, None, qc, qs, q_scale)
        return Nv4Act(qc, qs, q_scale, 0)
    if out is None:
        out = torch.empty(T, n_ff, dtype=torch.bfloat16, device=dev)
    C.wgemm_nv4(w.view2d(), w.sf, w.gscale, xq.codes, xq.sf, xq.gscale, xq.stride, out, None, None, None, n_ff, True,
                n_ff, a, bn, ws.status, None, None, None, None, 0, 0, T, None, None, None, None)
    return out


def pick_bn(n_tok: int, dual: bool) -> int:
    bn = 32
    cap = 128 if dual else 256
    while bn < n_tok and bn < cap:
        bn *= 2
    return bn


def _pick_split_k(n_tok_tiles: int, feat_tiles: int, K: int) -> int:
    """Split K when a skinny GEMM has too few tiles to keep the SMs streaming weights."""
    tiles = n_tok_tiles * feat_tiles
    num_kb = (K + 63) // 64
    if tiles >= NUM_SMS // 2 or num_kb < 8:
        return 1
    s = min(NUM_SMS // max(tiles, 1), num_kb // 4, 16)
    return max(1, s)


class Fp8Weight:
    """Block-scaled FP8 weight kept in its 8-bit encoding: ``data`` uint8 e4m3 bit patterns [..., rows, K] and
    ``scale`` float32 per 128 x 128 block [..., ceil(rows / 128), K / 128] (the layout of FP8 checkpoints with
    ``weight_block_size = [128, 128]``; ``weight_scale_inv`` is this scale). The GEMM feeds the bytes straight to
    the e4m3 tensor-core instruction, with the activations quantised per token and 128 columns, and adds each
    128-wide k block with its two scales in fp32 (``csrc/gemm_sm100.cu``, FP8 mode): a decode step reads one byte
    per weight instead of two."""
    __slots__ = ("data", "scale")

    def __init__(self, data, scale):
        self.data, self.scale = data.view(torch.uint8), scale.float().contiguous()

    @property
    def shape(self):
        return tuple(self.data.shape)

    @property
    def device(self):
        return self.data.device

    def dim(self):
        return self.data.dim()

    def view2d(self):
        return self.data.reshape(-1, self.data.shape[-1]), self.scale.reshape(-1, self.scale.shape[-1])

    def narrow(self, lo: int, hi: int) -> "Fp8Weight":
        return Fp8Weight(self.data[lo:hi], self.scale[lo:hi])

    def squeeze0(self) -> "Fp8Weight":
        return Fp8Weight(self.data[0], self.scale[0])

    @classmethod
    def quantize(cls, w: torch.Tensor):
        """Device-side encoding of a CUDA bf16 weight [..., rows, K] (rows a multiple of 128 when stacked)."""
        C = ext()
        rows, K = w.shape[-2], w.shape[-1]
        if K % 128 or (w.dim() > 2 and rows % 128):
            raise ValueError("FP8 block scaling needs K % 128 == 0 and 128-row aligned stacks")
        flat = w.reshape(-1, K).contiguous()
        data = torch.empty(flat.shape, dtype=torch.uint8, device=w.device)
        scale = torch.empty((flat.shape[0] + 127) // 128, K // 128, dtype=torch.float32, device=w.device)
        C.fp8_block_quant(flat, 128, 128, data, scale)
        lead = tuple(w.shape[:-2])
        return cls(data.view(*lead, rows, K), scale.view(*lead, (rows + 127) // 128, K // 128) if lead else scale)

    def dequantize(self, dtype=torch.bfloat16):
        C = ext()
        d2, s2 = self.view2d()
        out = torch.empty(d2.shape, dtype=torch.bfloat16, device=d2.device)
        C.fp8_block_dequant(d2.contiguous(), s2.contiguous(), 128, 128, out)
        return out.view(self.shape).to(dtype)


class Fp8Act:
    """Activation rows already encoded for the FP8 GEMMs (e4m3 bytes + one scale per row and 128 columns), kept with
    the bf16 rows they came from: a layer input that feeds several FP8 projections is encoded once."""
    __slots__ = ("x", "data", "scale")

    def __init__(self, x, data, scale):
        self.x, self.data, self.scale = x, data, scale

    is_cuda = True

    @property
    def shape(self):
        return self.x.shape

    @property
    def device(self):
        return self.x.device

    @classmethod
    def of(cls, x):
        d, s = fp8_quant_act(x)
        return cls(x, d, s)


def _fp8_parts(x):
    return (x.data, x.scale) if isinstance(x, Fp8Act) else fp8_quant_act(x)


def fp8_quant_act(x, out=None, scale=None):
    """bf16 activations [T, K] -> (e4m3 bytes [T, K], fp32 scale per row and 128 columns [T, K / 128])."""
    C = ext()
    T, K = x.shape
    if out is None:
        out = torch.empty(T, K, dtype=torch.uint8, device=x.device)
        scale = torch.empty(T, K // 128, dtype=torch.float32, device=x.device)
    C.fp8_act_quant(x, out, scale)
    return out, scale


def _linear_fp8(x, w: "Fp8Weight", residual, out, dual: bool, n_feat: int):
    C = ext()
    T, K = x.shape
    ws = Workspace.get(x.device)
    x8, xs = _fp8_parts(x)
    bn = 32 if T <= 32 else 64
    n_tt = (T + bn - 1) // bn
    ft = (n_feat + 127) // 128
    sk = _pick_split_k(n_tt, ft, K)
    if sk > 1:
        need = C.wgemm_workspace_floats(bn, dual, n_tt, ft, sk)
        if need > ws.splitk.numel() or n_tt * ft > ws.counters.numel():
            sk = 1
    w2, s2 = w.view2d()
    C.wgemm_fp8(w2, s2, x8, xs, out, residual, None, None, n_feat, dual, n_feat if dual else 0, bn, sk,
                ws.splitk if sk > 1 else None, ws.counters if sk > 1 else None, ws.status, None, None, None, None, 0, 0,
                T, None)
    return out


def linear(x, w, residual=None, out=None, out_dtype=torch.bfloat16, split_k: Optional[int] = None, bn=None):
    """out[T, N] = x[T, K] @ w[N, K]^T (+ residual)."""
    C = ext()
    if isinstance(x, Fp8Act) and not isinstance(w, Fp8Weight):
        x = x.x
    T, K = x.shape
    N = w.shape[0]
    q = isinstance(w, QWeight)
    if q and out_dtype != torch.bfloat16:
        raise ValueError("NVFP4 weights produce bf16 outputs")
    if out is None:
        out = torch.empty(T, N, dtype=out_dtype, device=x.device)
    if T == 0:
        return out
    if isinstance(w, Fp8Weight):
        if out_dtype != torch.bfloat16:
            raise ValueError("FP8 weights produce bf16 outputs")
        return _linear_fp8(x, w, residual, out, False, N)
    if isinstance(w, Nv4Weight):
        if out_dtype != torch.bfloat16:
            raise ValueError("NVFP4 weights produce bf16 outputs")
        return linear_nv4(x if isinstance(x, Nv4Act) else nv4_quant_act(x), w, residual=residual, out=out)
    ws = Workspace.get(x.device)
    bn = bn or pick_bn(T, False)
    n_tt = (T + bn - 1) // bn
    ft = (N + 127) // 128
    sk = _pick_split_k(n_tt, ft, K) if split_k is None else split_k
    if sk > 1:
        need = C.wgemm_workspace_floats(bn, False, n_tt, ft, sk)
        if need > ws.splitk.numel() or n_tt * ft > ws.counters.numel():
            sk = 1
    C.wgemm(w.codes if q else w, x, out, residual, None, None, N, False, 0, bn, sk, ws.splitk if sk > 1 else None,
            ws.counters if sk > 1 else None, ws.status, None, None, None, None, 0, 0, T, [], None,
            w.scales if q else None, w.gscale if q else None)
    return out


def gate_up_act(x, w_gate_up, n_ff: int, out=None, bn=None, split_k: Optional[int] = None):
    """silu(x @ Wg^T) * (x @ Wu^T) with Wg = w_gate_up[:n_ff], Wu = w_gate_up[n_ff:]."""
    C = ext()
    if isinstance(x, Fp8Act) and not isinstance(w_gate_up, Fp8Weight):
        x = x.x
    T, K = x.shape
    if out is None:
        out = torch.empty(T, n_ff, dtype=torch.bfloat16, device=x.device)
    if T == 0:
        return out
    if isinstance(w_gate_up, Fp8Weight):
        return _linear_fp8(x, w_gate_up, None, out, True, n_ff)
    if isinstance(w_gate_up, Nv4Weight):
        return gate_up_nv4(x if isinstance(x, Nv4Act) else nv4_quant_act(x), w_gate_up, n_ff, out=out)
    ws = Workspace.get(x.device)
    bn = bn or pick_bn(T, True)
    n_tt = (T + bn - 1) // bn
    ft = (n_ff + 127) // 128
    sk = _pick_split_k(n_tt, ft, K) if split_k is None else split_k
    if sk > 1:
        need = C.wgemm_workspace_floats(bn, True, n_tt, ft, sk)
        if need > ws.splitk.numel() or n_tt * ft > ws.counters.numel():
            sk = 1
    q = isinstance(w_gate_up, QWeight)
    C.wgemm(w_gate_up.codes if q else w_gate_up, x, out, None, None, None, n_ff, True, n_ff, bn, sk,
            ws.splitk if sk > 1 else None, ws.counters if sk > 1 else None, ws.status, None, None, None, None, 0, 0, T,
            [], None, w_gate_up.scales if q else None, w_gate_up.gscale if q else None)
    return out


def rmsnorm(x, w, eps, w_offset=0.0, residual=None, out=None, sum_out=None):
    """Returns (normed, summed). With a residual the sum x + residual is the new residual stream."""
    C = ext()
    if out is None:
        out = torch.empty_like(x)
    if residual is not None and sum_out is None:
        sum_out = torch.empty_like(x)
    C.rmsnorm(x, residual, sum_out, w, out, eps, w_offset)
    return out, (sum_out if residual is not None else x)


def qk_norm_rope_append(qkv, n_q, n_kv, d, q_norm_w, k_norm_w, eps, w_offset, cos_sin, rot, positions, slots,
                        k_cache, v_cache, gated_q=False, q_out=None):
    C = ext()
    T = qkv.shape[0]
    if q_out is None:
        q_out = torch.empty(T, n_q, d, dtype=torch.bfloat16, device=qkv.device)
    qhs = 2 * d if gated_q else d
    k_off = n_q * qhs
    v_off = k_off + n_kv * d
    C.qk_norm_rope_append(qkv, qhs, k_off, v_off, q_norm_w, k_norm_w, eps, w_offset, cos_sin, rot, positions, slots,
                          q_out, k_cache, v_cache, n_q, n_kv, d)
    return q_out


def sigmoid_gate(attn, qkv, n_q, d, out=None):
    C = ext()
    if out is None:
        out = torch.empty_like(attn)
    C.sigmoid_gate(attn, qkv, 2 * d, d, n_q, out)
    return out


def decode_splits(batch: int, n_kv_heads: int, g_tiles: int, max_ctx: int, head_dim: int = 128) -> int:
    """Flash-decoding split count. The grid is (batch x kv heads x head tiles x splits) CTAs, one resident per SM
    (its K/V rings take most of the shared memory), and a split covers ceil(tiles / splits) 128-key tiles. The
    count minimises waves x (tiles per split + fixed cost per CTA): 2.2 waves cost as much as 3, and a count
    that leaves the last split empty only adds idle CTAs."""
    ctas = max(1, batch * n_kv_heads * g_tiles)
    slots = NUM_SMS
    tiles = max(1, (max_ctx + 127) // 128)
    fixed = TUNE["decode_fixed_tiles"]
    best, best_cost = 1, None
    for s in range(1, min(128, tiles) + 1):
        per = (tiles + s - 1) // s
        if (tiles + per - 1) // per != s:
            continue
        waves = (ctas * s + slots - 1) // slots
        cost = waves * (per + fixed)
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


def paged_decode(q, k_cache, v_cache, block_table, ctx_lens, scale, window=0, n_splits=None, max_ctx=None, out=None,
                 impl="tc"):
    C = ext()
    B, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    if n_splits is None:
        G = Hq // Hkv
        n_splits = decode_splits(B, Hkv, (G + 15) // 16, max_ctx or block_table.shape[1] * k_cache.shape[1], D)
    ws = Workspace.get(q.device)
    o_part = ws.buf("dec_o", (B * Hq * n_splits * 2 * D,), torch.float32)
    ml_part = ws.buf("dec_ml", (B * Hq * n_splits * 2 * 2,), torch.float32)
    if out is None:
        out = torch.empty_like(q)
    C.paged_decode(q, k_cache, v_cache, block_table, ctx_lens, scale, window, n_splits, o_part, ml_part, out,
                   impl == "tc", ws.status, ws.counters)
    return out


def prefill_attn(q, k_cache, v_cache, cu_q, ctx_lens, block_table, max_q_len, scale, window=0, causal=True, out=None):
    C = ext()
    if out is None:
        out = torch.empty_like(q)
    ws = Workspace.get(q.device)
    C.prefill_attn(q, k_cache, v_cache, cu_q, ctx_lens, block_table, max_q_len, scale, window, causal, out, ws.status)
    return out


def head_linear(x, w2d, n_heads: int, rows_per_group: int, n_feat: int, K: int, x_group_col: int, out2d):
    """Per-head projections read and written in place: for every head h
    ``out2d[t * n_heads + h, :n_feat] = W_h @ x[t, h * x_group_col : h * x_group_col + K]`` with
    ``W_h = w2d[h * rows_per_group : h * rows_per_group + n_feat]``. One grouped launch of the tcgen05 GEMM (group =
    head); the activation tile of a head is fetched from its column slice of ``x`` by the TMA load, the output rows
    go through a row map, so nothing is transposed or copied."""
    C = ext()
    T = x.shape[0]
    ws = Workspace.get(x.device)
    bn = pick_bn(T, False)
    key = ("head_linear", T, n_heads, bn)
    tab = ws._cache.get(key)
    if tab is None:
        n_tt = (T + bn - 1) // bn
        Tp = n_tt * bn
        h = torch.arange(n_heads).repeat_interleave(n_tt)
        tt = torch.arange(n_tt).repeat(n_heads)
        rows = torch.full((n_heads * Tp,), -1, dtype=torch.int32)
        t = torch.arange(T)
        for hh in range(n_heads):
            rows[hh * Tp: hh * Tp + T] = (t * n_heads + hh).int()
        i32 = dict(dtype=torch.int32, device=x.device)
        tab = (h.to(**i32), (tt * bn).to(**i32), torch.clamp(T - tt * bn, max=bn).to(**i32),
               (h * Tp + tt * bn).to(**i32), rows.to(x.device),
               torch.tensor([n_heads * n_tt, 0], **i32), n_heads * n_tt)
        ws._cache[key] = tab
    tile_group, tile_tok0, tile_ntok, tile_out0, out_rows, meta, n_tiles = tab
    C.wgemm(w2d, x, out2d, None, None, out_rows, n_feat, False, 0, bn, 1, None, None, ws.status, tile_group, tile_tok0,
            tile_ntok, meta, n_tiles, rows_per_group, 0, [], tile_out0, None, None, x_group_col, K)
    return out2d


def mla_splits(n_seqs: int, max_q_len: int, nh: int, max_ctx: int) -> int:
    """Key splits of the latent-attention kernel: enough CTAs (64 query rows each) to cover the SMs, at least four
    64-key tiles per split."""
    g = min(nh, 64)
    tiles = max(1, n_seqs * ((max_q_len + 64 // g - 1) // (64 // g)) * max(1, nh // 64))
    by_sm = max(1, NUM_SMS // tiles)
    by_len = max(1, (max_ctx + 255) // 256)
    return int(max(1, min(by_sm, by_len, 32)))


def mla_supported(nh: int, kv_lora: int, rope_dim: int, page: int) -> bool:
    return kv_lora == 512 and rope_dim == 64 and page % 8 == 0 and 64 % page == 0 and \
        ((nh >= 64 and nh % 64 == 0) or (0 < nh < 64 and 64 % nh == 0))


def mla_prep(kva, norm_w, eps, w_offset, q, q_pe_off, cos_sin, positions, slots, cache, q_abs):
    """Cache row [rmsnorm(c_kv) | rope(k_pe)] written at each token's cell and rope(q_pe) written into
    q_abs[..., 512:] in one launch."""
    ext().mla_prep(kva, norm_w, eps, w_offset, q, q_pe_off, cos_sin, positions, slots, cache, q_abs)


def mla_attn(q_abs, cache, cu_q, ctx_lens, block_table, page, max_q_len, scale, n_splits=None, max_ctx=None, out=None):
    """Latent attention, absorbed form: q_abs [T, heads, 576], cache rows [.., 576] -> [T, heads, 512]."""
    C = ext()
    T, nh, _ = q_abs.shape
    if n_splits is None:
        n_splits = mla_splits(int(ctx_lens.numel()), max_q_len, nh, max_ctx or block_table.shape[1] * page)
    ws = Workspace.get(q_abs.device)
    o_part = ml_part = None
    if n_splits > 1:
        o_part = ws.buf("mla_o", (T * nh * n_splits * 512,), torch.float32)
        ml_part = ws.buf("mla_ml", (T * nh * n_splits * 2,), torch.float32)
    if out is None:
        out = torch.empty(T, nh, 512, dtype=torch.bfloat16, device=q_abs.device)
    C.mla_attn(q_abs, cache, cu_q, ctx_lens, block_table, page, max_q_len, scale, n_splits, o_part, ml_part, out,
               ws.status)
    return out


def router_topk(logits, k, mode="softmax", renorm=True, route_scale=1.0, bias=None, n_group=1, topk_group=1,
                ids=None, wts=None):
    C = ext()
    T = logits.shape[0]
    if ids is None:
        ids = torch.empty(T, k, dtype=torch.int32, device=logits.device)
        wts = torch.empty(T, k, dtype=torch.float32, device=logits.device)
    C.router_topk(logits, bias, k, 0 if mode == "softmax" else 1, renorm, route_scale, n_group, topk_group, ids, wts)
    return ids, wts


class Routing:
    """Router result of one step: ``ids`` / ``wts`` [T, k] and, for decode-sized steps, the dense routing tables
    (``dense``) that let the expert GEMMs run without a gather. Unpacks as ``ids, wts = routing``."""
    __slots__ = ("ids", "wts", "dense", "x_normed", "e_lo", "n_local", "shared_slot", "xq")

    def __init__(self, ids, wts, dense=None, x_normed=None, e_lo=0, n_local=None):
        self.ids, self.wts, self.dense, self.x_normed = ids, wts, dense, x_normed
        self.e_lo, self.n_local = e_lo, n_local      # expert range the dense tables were built for
        self.shared_slot = False                     # the shared expert has a slot of its own in the dense tables
        self.xq = None                               # the experts' input already NVFP4-encoded (Nv4Act)

    def __iter__(self):
        yield self.ids
        yield self.wts


class DenseRoute:
    """Device tables of the dense routing (one token tile per active expert covering all T tokens). ``bn`` is the
    token tile of the GEMMs, ``stride`` the distance between the rows of consecutive slots in the intermediate
    tensor (= bn, or 128 for the NVFP4 path whose 32-token tiles must start a 128-row scale atom), ``n_slots`` the
    most slots a step can have (local experts, + 1 when the shared expert is stacked behind them)."""

    def __init__(self, n_slots: int, bn: int, device, stride: Optional[int] = None):
        i32 = dict(dtype=torch.int32, device=device)
        self.n_slots, self.bn, self.stride = n_slots, bn, stride or bn
        self.E = n_slots
        self.tile_group = torch.zeros(n_slots, **i32)
        self.slot_base = torch.zeros(n_slots, **i32)
        self.zeros = torch.zeros(n_slots, **i32)
        self.tile_ntok = torch.zeros(n_slots, **i32)
        self.meta = torch.zeros(2, **i32)
        self.out_rows = torch.full((n_slots * self.stride,), -1, **i32)
        self.tok_scale = torch.zeros(n_slots * self.stride, dtype=torch.float32, device=device)
        self.h8 = self.h8_scale = None               # FP8 experts: the activated rows, encoded by the gate/up GEMM
        self.sh_logit = torch.zeros(4 * 64, dtype=torch.float32, device=device)   # one plane per column split
        self.active = torch.zeros(n_slots, **i32)      # per local expert: chosen by some token of the step
        self.h_all = None
        self.hq = None
        self.y_pairs = None


def router(x, w_router, k, mode="softmax", renorm=True, route_scale=1.0, bias=None, n_group=1, topk_group=1,
           norm=None, e_lo: int = 0, n_local: Optional[int] = None, slot_stride: Optional[int] = None, sh_gate=None,
           shared_slot: bool = False):
    """Router logits and top-k selection -> ``Routing``. Decode-sized steps (<= 64 tokens, <= 1024 pairs) run as
    ONE launch that also builds the dense routing tables; with ``norm=(weight, eps, w_offset)`` that launch first
    applies the RMSNorm to ``x`` (the raw residual stream) and ``Routing.x_normed`` is the normalised input.
    ``shared_slot``: the shared expert is stacked behind the local routed experts and gets a slot of its own that
    every token uses (weight sigmoid(x . sh_gate) when ``sh_gate`` [1, H] is given, else 1); its output rows are
    the pairs T * k .. T * k + T - 1. Larger steps use the GEMM and the selection kernel."""
    T, E = x.shape[0], w_router.shape[0]
    small = T <= 64 and T * k <= 1024 and TUNE["fused_router"]
    if not small:
        xn = None
        if norm is not None:
            xn, _ = rmsnorm(x, norm[0], norm[1], norm[2])
        logits = linear(x if xn is None else xn, w_router, out_dtype=torch.float32)
        ids, wts = router_topk(logits, k, mode, renorm, route_scale, bias, n_group, topk_group)
        return Routing(ids, wts, None, xn)
    C = ext()
    ws = Workspace.get(x.device)
    logits = ws.buf("router_logits", (4 * 64 * 512,), torch.float32)    # one plane per column split
    ctr = ws._cache.get("router_ctr")
    if ctr is None:
        ctr = torch.zeros(4, dtype=torch.int32, device=x.device)
        ws._cache["router_ctr"] = ctr
    bn = 32 if T <= 32 else 64
    stride = slot_stride or bn
    nl = E if n_local is None else n_local
    n_slots = nl + (1 if shared_slot else 0)
    dr = ws._cache.get(("dense_route", n_slots, bn, stride))
    if dr is None:
        dr = DenseRoute(n_slots, bn, x.device, stride)
        ws._cache[("dense_route", n_slots, bn, stride)] = dr
    ids = torch.empty(T, k, dtype=torch.int32, device=x.device)
    wts = torch.empty(T, k, dtype=torch.float32, device=x.device)
    xn = torch.empty_like(x) if norm is not None else None
    C.moe_route_small(x, norm[0] if norm else None, norm[1] if norm else 0.0, norm[2] if norm else 0.0, xn, w_router,
                      bias, k, 0 if mode == "softmax" else 1, renorm, route_scale, n_group, topk_group, logits, ids, wts,
                      stride, dr.tile_group, dr.slot_base, dr.tile_ntok, dr.meta, dr.out_rows, dr.tok_scale, ctr,
                      e_lo, nl, sh_gate.reshape(-1) if sh_gate is not None else None,
                      dr.sh_logit if sh_gate is not None else None, bool(shared_slot), ws.status, dr.active)
    r = Routing(ids, wts, dr, xn, e_lo, nl)
    r.shared_slot = bool(shared_slot)
    return r


class MoePlan:
    """Device buffers of one routing plan (sized for the largest step; reused every step)."""

    def __init__(self, max_tokens: int, k: int, n_local: int, bn: int, device):
        P = max_tokens * k
        i32 = dict(dtype=torch.int32, device=device)
        self.max_tokens, self.k, self.n_local, self.bn = max_tokens, k, n_local, bn
        self.max_tiles = (P + bn - 1) // bn + n_local
        self.counts = torch.zeros(n_local, **i32)
        self.offsets = torch.zeros(n_local + 1, **i32)
        self.sorted_token = torch.zeros(P, **i32)
        self.sorted_pair = torch.zeros(P, **i32)
        self.sorted_w = torch.zeros(P, dtype=torch.float32, device=device)
        self.tile_group = torch.zeros(self.max_tiles, **i32)
        self.tile_tok0 = torch.zeros(self.max_tiles, **i32)
        self.tile_ntok = torch.zeros(self.max_tiles, **i32)
        self.meta = torch.zeros(2, **i32)  # {n_tiles, n_rows}
        self.x_sorted = None
        self.h_sorted = None
        self.y_pairs = None


def _dense_ok(routing, n_groups: int, e_lo: int, ids) -> bool:
    return (routing is not None and routing.dense is not None and routing.e_lo == e_lo and routing.ids is ids
            and routing.n_local + int(routing.shared_slot) == n_groups and bool(TUNE["dense_route"]))


def _dense_pairs(dr: DenseRoute, P: int, T: int, k: int, H: int, device):
    """Output rows of the down projection: one per (token, expert) pair, then one per token for the shared slot."""
    if dr.y_pairs is None or dr.y_pairs.shape[0] < P + T or dr.y_pairs.shape[1] != H:
        dr.y_pairs = torch.zeros(max(P, 64 * k) + 64, H, dtype=torch.bfloat16, device=device)
    return dr.y_pairs


class PendingCombine:
    """The weighted pair rows of a decode-sized MoE layer whose per-token sum has not run yet: the rank-partial
    result of an expert-parallel layer, handed to the reduction that follows so that it sums them inside its own
    launch (``parallel.symm.SymmComm.all_reduce_add_norm``). ``materialize`` runs the combine kernel instead."""
    __slots__ = ("y", "ids", "e_lo", "e_hi", "shared", "T", "H")

    def __init__(self, y, ids, e_lo, e_hi, shared, T, H):
        self.y, self.ids, self.e_lo, self.e_hi, self.shared, self.T, self.H = y, ids, e_lo, e_hi, shared, T, H

    def materialize(self, out=None):
        if out is None:
            out = torch.empty(self.T, self.H, dtype=torch.bfloat16, device=self.y.device)
        ext().moe_combine(self.y, self.ids, self.e_lo, self.e_hi, self.shared, None, None, out, None, 0.0, 0.0, None)
        return out


def _dense_combine(dr: DenseRoute, routing, ids, e_lo, T, k, H, shared, shared_gate, residual, out, norm, device,
                   defer: bool = False):
    C = ext()
    P = T * k
    y = dr.y_pairs[:P]
    if routing.shared_slot:
        # the shared expert ran as a slot of the grouped GEMMs; its gate is already applied
        shared, shared_gate = dr.y_pairs[P:P + T], None
    if defer and shared_gate is None and residual is None and norm is None:
        return PendingCombine(y, ids, e_lo, e_lo + routing.n_local, shared, T, H)
    if out is None:
        out = torch.empty(T, H, dtype=torch.bfloat16, device=device)
    if norm is None:
        C.moe_combine(y, ids, e_lo, e_lo + routing.n_local, shared, shared_gate, residual, out, None, 0.0, 0.0, None)
        return out
    normed = torch.empty(T, H, dtype=torch.bfloat16, device=device)
    C.moe_combine(y, ids, e_lo, e_lo + routing.n_local, shared, shared_gate, residual, out, norm[0], norm[1], norm[2],
                  normed)
    return out, normed


def _moe_experts_nv4(x, ids, wts, w_gate_up: "Nv4Weight", w_down: "Nv4Weight", n_ff, e_lo, shared, shared_gate,
                     residual, out, norm, routing, xq: Optional["Nv4Act"] = None, h_scale=None, defer: bool = False):
    """Routed experts on the native NVFP4 path (decode-sized steps over the dense routing): the layer input is
    quantised once (or arrives quantised as ``xq``), the gate/up GEMM re-encodes its SwiGLU output to NVFP4 in its
    epilogue (static tensor scale ``h_scale``), and the down GEMM reads that. Three launches + the combine."""
    C = ext()
    T, H = x.shape
    k = ids.shape[1]
    n_groups = w_gate_up.shape[0]
    ws = Workspace.get(x.device)
    dr = routing.dense
    P = T * k
    if xq is None:
        xq = nv4_quant_act(x, key="moe_x")
    if h_scale is None:
        h_scale = _nv4_h_scale(ws, x.device)
    rows = dr.n_slots * dr.stride
    if dr.hq is None or dr.hq[0].shape[1] * 2 != n_ff:
        dr.hq = (torch.zeros(rows, n_ff // 2, dtype=torch.uint8, device=x.device),
                 torch.zeros(C.nv4_sf_bytes(rows, n_ff), dtype=torch.uint8, device=x.device))
    hq_codes, hq_sf = dr.hq
    y_pairs = _dense_pairs(dr, P, T, k, H, x.device)
    C.wgemm_nv4(w_gate_up.view2d(), w_gate_up.sf, w_gate_up.gscale, xq.codes, xq.sf, xq.gscale, xq.stride, None, None,
                None, None, n_ff, True, n_ff, 0, dr.bn, ws.status, dr.tile_group, dr.zeros, dr.tile_ntok, dr.meta,
                dr.n_slots, 2 * n_ff, 0, dr.slot_base, hq_codes, hq_sf, h_scale)
    C.wgemm_nv4(w_down.view2d(), w_down.sf, w_down.gscale, hq_codes, hq_sf, h_scale, 0, y_pairs, None, dr.tok_scale,
                dr.out_rows, H, False, 0, 0, dr.bn, ws.status, dr.tile_group, dr.slot_base, dr.tile_ntok, dr.meta,
                dr.n_slots, H, 0, None, None, None, None)
    return _dense_combine(dr, routing, ids, e_lo, T, k, H, shared, shared_gate, residual, out, norm, x.device, defer)


class Nv4Plan:
    """Routing plan and expert-sorted NVFP4 buffers of a prompt-sized step on the native path: every expert's rows
    start on a token-tile boundary (``bn`` rows) so the tile's scale factors start where the tensor-core copy
    wants them."""

    def __init__(self, max_tokens: int, k: int, n_local: int, bn: int, H: int, n_ff: int, device):
        C = ext()
        P = max_tokens * k
        i32 = dict(dtype=torch.int32, device=device)
        u8 = dict(dtype=torch.uint8, device=device)
        self.bn = bn
        self.rows = (P + n_local * bn + 127) // 128 * 128
        self.max_tiles = (P + bn - 1) // bn + n_local
        self.counts2 = torch.zeros(2 * n_local, **i32)
        self.offsets = torch.zeros(n_local + 1, **i32)
        self.sorted_token = torch.full((self.rows,), -1, **i32)
        self.sorted_pair = torch.zeros(self.rows, **i32)
        self.sorted_w = torch.zeros(self.rows, dtype=torch.float32, device=device)
        self.tile_group = torch.zeros(self.max_tiles, **i32)
        self.tile_tok0 = torch.zeros(self.max_tiles, **i32)
        self.tile_ntok = torch.zeros(self.max_tiles, **i32)
        self.meta = torch.zeros(2, **i32)
        self.x_codes = torch.zeros(self.rows, H // 2, **u8)
        self.x_sf = torch.zeros(C.nv4_sf_bytes(self.rows, H), **u8)
        self.x_gs = torch.ones(self.rows, dtype=torch.float32, device=device)
        self.h_codes = torch.zeros(self.rows, n_ff // 2, **u8)
        self.h_sf = torch.zeros(C.nv4_sf_bytes(self.rows, n_ff), **u8)
        self.y_pairs = torch.zeros(P, H, dtype=torch.bfloat16, device=device)


def _nv4_h_scale(ws, device):
    h_scale = ws._cache.get("nv4_h_scale")
    if h_scale is None:
        h_scale = torch.tensor([NV4_H_AMAX / (6.0 * 448.0)], dtype=torch.float32, device=device)
        ws._cache["nv4_h_scale"] = h_scale
    return h_scale


def _moe_experts_nv4_sorted(x, ids, wts, w_gate_up: "Nv4Weight", w_down: "Nv4Weight", n_ff, e_lo, shared, shared_gate,
                            residual, out, norm, xq: Optional["Nv4Act"] = None):
    """Routed experts of a prompt-sized step on the native NVFP4 path: the tokens are encoded once, their codes and
    scale bytes are gathered into expert order (aligned segments), the gate/up GEMM re-encodes its SwiGLU output
    and the down GEMM scatters weighted rows to their pairs. Nothing is expanded to bf16 on the way."""
    C = ext()
    T, H = x.shape
    k = ids.shape[1]
    E_local = w_gate_up.shape[0]
    ws = Workspace.get(x.device)
    bn = TUNE["nv4_sorted_bn"]
    cap = 1024
    while cap < T:
        cap *= 2
    key = ("nv4_plan", cap, k, E_local, bn, H, n_ff)
    plan = ws._cache.get(key)
    if plan is None:
        plan = Nv4Plan(cap, k, E_local, bn, H, n_ff, x.device)
        ws._cache[key] = plan
    C.moe_plan_aligned(ids, wts, e_lo, E_local, bn, bn, plan.counts2, plan.offsets, plan.sorted_token,
                       plan.sorted_pair, plan.sorted_w, plan.tile_group, plan.tile_tok0, plan.tile_ntok, plan.meta)
    if xq is None:
        xq = nv4_quant_act(x, key="moe_x_big")
    C.nv4_gather_rows(xq.codes, xq.sf, xq.gscale if xq.stride else None, plan.sorted_token, plan.meta[1:2],
                      plan.x_codes, plan.x_sf, plan.x_gs if xq.stride else None)
    h_scale = _nv4_h_scale(ws, x.device)
    C.wgemm_nv4(w_gate_up.view2d(), w_gate_up.sf, w_gate_up.gscale, plan.x_codes, plan.x_sf,
                plan.x_gs if xq.stride else xq.gscale, 1 if xq.stride else 0, None, None, None, None, n_ff, True, n_ff,
                0, bn, ws.status, plan.tile_group, plan.tile_tok0, plan.tile_ntok, plan.meta, plan.max_tiles, 2 * n_ff,
                0, None, plan.h_codes, plan.h_sf, h_scale)
    C.wgemm_nv4(w_down.view2d(), w_down.sf, w_down.gscale, plan.h_codes, plan.h_sf, h_scale, 0, plan.y_pairs, None,
                plan.sorted_w, plan.sorted_pair, H, False, 0, 0, bn, ws.status, plan.tile_group, plan.tile_tok0,
                plan.tile_ntok, plan.meta, plan.max_tiles, H, 0, None, None, None, None)
    if out is None:
        out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    if norm is None:
        C.moe_combine(plan.y_pairs, ids, e_lo, e_lo + E_local, shared, shared_gate, residual, out, None, 0.0, 0.0, None)
        return out
    normed = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    C.moe_combine(plan.y_pairs, ids, e_lo, e_lo + E_local, shared, shared_gate, residual, out, norm[0], norm[1],
                  norm[2], normed)
    return out, normed


# largest |SwiGLU output| the static scale of the re-encoded intermediate is laid out for (checkpoints bring their
# own calibrated input scale; this is the default for weights quantised here)
NV4_H_AMAX = 32.0


def moe_experts(x, ids, wts, w_gate_up, w_down, n_ff, e_lo=0, plan: Optional[MoePlan] = None, shared=None,
                shared_gate=None, residual=None, out=None, norm=None, routing: Optional[Routing] = None,
                defer_combine: bool = False):
    """Routed experts over the device routing plan: plan -> gather -> grouped gate/up (+SwiGLU) ->
    grouped down (x routing weight) -> combine (+ shared expert, + residual).

    w_gate_up: [E_local, 2*n_ff, H]; w_down: [E_local, H, n_ff]; ids/wts: [T, k]. Returns bf16 [T, H]; with
    ``norm=(weight, eps, w_offset)`` the combine also applies that RMSNorm and (out, normed) is returned."""
    C = ext()
    T, H = x.shape
    k = ids.shape[1]
    E_local = w_gate_up.shape[0]
    ws = Workspace.get(x.device)
    if isinstance(w_gate_up, Fp8Weight):
        return _moe_experts_fp8(x, ids, wts, w_gate_up, w_down, n_ff, e_lo, shared, shared_gate, residual, out, norm,
                                routing, defer=defer_combine)
    if isinstance(w_gate_up, Nv4Weight):
        if _dense_ok(routing, E_local, e_lo, ids):
            return _moe_experts_nv4(x, ids, wts, w_gate_up, w_down, n_ff, e_lo, shared, shared_gate, residual, out,
                                    norm, routing, xq=routing.xq, defer=defer_combine)
        wfp4_ok = H % 256 == 0 and n_ff % 256 == 0       # what the de-quantising GEMM needs of K
        if (TUNE["nv4_sorted"] and (T * k >= 64 * E_local or not wfp4_ok)
                and not (routing is not None and routing.shared_slot)):
            return _moe_experts_nv4_sorted(x, ids, wts, w_gate_up, w_down, n_ff, e_lo, shared, shared_gate, residual,
                                           out, norm, xq=routing.xq if routing is not None else None)
        # steps in between: the de-quantising grouped GEMM over the routing plan (same codes, linear scale order)
        w_gate_up, w_down = w_gate_up.as_qweight(), w_down.as_qweight()
    if routing is not None and routing.shared_slot and not _dense_ok(routing, E_local, e_lo, ids):
        raise ValueError("the routing carries a shared-expert slot that these expert weights do not have")
    if routing is None or not routing.shared_slot:
        n_routed = E_local
    else:
        n_routed = E_local - 1
    # expert weights as 2-D operands (+ NVFP4 block scales / tensor scales when kept in 4 bits)
    if isinstance(w_gate_up, QWeight):
        (gu2, gu_sc), gu_gs = w_gate_up.view2d(), w_gate_up.gscale
    else:
        gu2, gu_sc, gu_gs = w_gate_up.view(E_local * 2 * n_ff, H), None, None
    if isinstance(w_down, QWeight):
        (dn2, dn_sc), dn_gs = w_down.view2d(), w_down.gscale
    else:
        dn2, dn_sc, dn_gs = w_down.view(E_local * H, n_ff), None, None
    if _dense_ok(routing, E_local, e_lo, ids):
        # decode-sized step: every active expert runs over all T tokens in place (no plan, no gather)
        dr = routing.dense
        P = T * k
        if dr.h_all is None or dr.h_all.shape[1] != n_ff:
            dr.h_all = torch.zeros(dr.n_slots * dr.stride, n_ff, dtype=torch.bfloat16, device=x.device)
        y_pairs = _dense_pairs(dr, P, T, k, H, x.device)
        C.wgemm(gu2, x, dr.h_all, None, None, None, n_ff, True, n_ff, dr.bn, 1,
                None, None, ws.status, dr.tile_group, dr.zeros, dr.tile_ntok, dr.meta, dr.n_slots, 2 * n_ff, 0, [],
                dr.slot_base, gu_sc, gu_gs)
        C.wgemm(dn2, dr.h_all, y_pairs, None, dr.tok_scale, dr.out_rows, H, False, 0,
                dr.bn, 1, None, None, ws.status, dr.tile_group, dr.slot_base, dr.tile_ntok, dr.meta, dr.n_slots, H, 0, [],
                None, dn_sc, dn_gs)
        return _dense_combine(dr, routing, ids, e_lo, T, k, H, shared, shared_gate, residual, out, norm, x.device,
                              defer_combine)
    E_local = n_routed
    if plan is None:
        bn = 32 if T * k <= 32 * E_local else (64 if T * k <= 64 * E_local else 128)
        key = ("moe_plan", T, k, E_local, bn, H, n_ff)
        plan = ws._cache.get(key)
        if plan is None:
            plan = MoePlan(T, k, E_local, bn, x.device)
            ws._cache[key] = plan
    P = T * k
    bn = plan.bn
    if (plan.x_sorted is None or plan.x_sorted.shape[0] < P + bn or plan.x_sorted.shape[1] != H
            or plan.h_sorted.shape[1] != n_ff):
        # padded by one tile so a tile that starts near the end stays inside the tensor map's rows
        plan.x_sorted = torch.zeros(P + bn, H, dtype=torch.bfloat16, device=x.device)
        plan.h_sorted = torch.zeros(P + bn, n_ff, dtype=torch.bfloat16, device=x.device)
        plan.y_pairs = torch.zeros(P, H, dtype=torch.bfloat16, device=x.device)
    if P <= 1024 and E_local <= 512 and TUNE["fused_plan"]:
        # decode-sized step: plan and gather in one launch
        C.moe_plan_gather(ids, wts, e_lo, E_local, bn, plan.counts, plan.offsets, plan.sorted_token,
                          plan.sorted_pair, plan.sorted_w, plan.tile_group, plan.tile_tok0, plan.tile_ntok, plan.meta,
                          x, plan.x_sorted)
    else:
        C.moe_plan(ids, wts, e_lo, E_local, bn, plan.counts, plan.offsets, plan.sorted_token, plan.sorted_pair,
                   plan.sorted_w, plan.tile_group, plan.tile_tok0, plan.tile_ntok, plan.meta)
        C.gather_rows(x, plan.sorted_token, plan.meta[1:2], plan.x_sorted[:P])
    C.wgemm(gu2, plan.x_sorted, plan.h_sorted, None, None, None, n_ff, True, n_ff, bn, 1, None, None, ws.status,
            plan.tile_group, plan.tile_tok0, plan.tile_ntok, plan.meta, plan.max_tiles, 2 * n_ff, 0, [], None,
            gu_sc, gu_gs)
    C.wgemm(dn2, plan.h_sorted, plan.y_pairs, None, plan.sorted_w, plan.sorted_pair, H, False, 0, bn, 1, None, None,
            ws.status, plan.tile_group, plan.tile_tok0, plan.tile_ntok, plan.meta, plan.max_tiles, H, 0, [], None,
            dn_sc, dn_gs)
    if out is None:
        out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    if norm is None:
        C.moe_combine(plan.y_pairs, ids, e_lo, e_lo + E_local, shared, shared_gate, residual, out, None, 0.0, 0.0, None)
        return out
    normed = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    C.moe_combine(plan.y_pairs, ids, e_lo, e_lo + E_local, shared, shared_gate, residual, out, norm[0], norm[1],
                  norm[2], normed)
    return out, normed


def _moe_experts_fp8(x, ids, wts, w_gate_up, w_down, n_ff, e_lo, shared, shared_gate, residual, out, norm, routing,
                     defer: bool = False):
    """Routed experts with block-scaled FP8 weights: the same two grouped GEMMs in FP8 mode; activations (the
    layer input and the SwiGLU output) are quantised per row and 128 columns before each of them."""
    C = ext()
    T, H = x.shape
    k = ids.shape[1]
    E_local = w_gate_up.shape[0]
    ws = Workspace.get(x.device)
    gu2, gu_s = w_gate_up.view2d()
    dn2, dn_s = w_down.view2d()
    P = T * k
    if out is None:
        out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    if _dense_ok(routing, E_local, e_lo, ids):
        dr = routing.dense
        if dr.h_all is None or dr.h_all.shape[1] != n_ff:
            dr.h_all = torch.zeros(dr.n_slots * dr.stride, n_ff, dtype=torch.bfloat16, device=x.device)
        y_pairs = _dense_pairs(dr, P, T, k, H, x.device)
        x8, xs = _fp8_parts(routing.xq) if isinstance(routing.xq, Fp8Act) else fp8_quant_act(x)
        if TUNE["fp8_fused_quant"] and n_ff % 128 == 0:
            # the gate/up epilogue encodes the activated rows itself (rows past a slot's tokens stay zero bytes)
            if dr.h8 is None or dr.h8.shape[1] != n_ff:
                dr.h8 = torch.zeros(dr.n_slots * dr.stride, n_ff, dtype=torch.uint8, device=x.device)
                dr.h8_scale = torch.ones(dr.n_slots * dr.stride, n_ff // 128, dtype=torch.float32, device=x.device)
            h8, hs = dr.h8, dr.h8_scale
            C.wgemm_fp8_q(gu2, gu_s, x8, xs, dr.h_all, None, None, None, n_ff, True, n_ff, dr.bn, 1, None, None,
                          ws.status, dr.tile_group, dr.zeros, dr.tile_ntok, dr.meta, dr.n_slots, 2 * n_ff, 0,
                          dr.slot_base, h8, hs)
        else:
            C.wgemm_fp8(gu2, gu_s, x8, xs, dr.h_all, None, None, None, n_ff, True, n_ff, dr.bn, 1, None, None,
                        ws.status, dr.tile_group, dr.zeros, dr.tile_ntok, dr.meta, dr.n_slots, 2 * n_ff, 0, dr.slot_base)
            h8, hs = fp8_quant_act(dr.h_all)
        C.wgemm_fp8(dn2, dn_s, h8, hs, y_pairs, None, dr.tok_scale, dr.out_rows, H, False, 0, dr.bn, 1, None, None,
                    ws.status, dr.tile_group, dr.slot_base, dr.tile_ntok, dr.meta, dr.n_slots, H, 0, None)
        return _dense_combine(dr, routing, ids, e_lo, T, k, H, shared, shared_gate, residual, out, norm, x.device,
                              defer=defer)
    if True:
        bn = 32 if P <= 32 * E_local else 64
        key = ("moe_plan", T, k, E_local, bn, H, n_ff)
        plan = ws._cache.get(key)
        if plan is None:
            plan = MoePlan(T, k, E_local, bn, x.device)
            ws._cache[key] = plan
        if (plan.x_sorted is None or plan.x_sorted.shape[0] < P + bn or plan.x_sorted.shape[1] != H
                or plan.h_sorted.shape[1] != n_ff):
            plan.x_sorted = torch.zeros(P + bn, H, dtype=torch.bfloat16, device=x.device)
            plan.h_sorted = torch.zeros(P + bn, n_ff, dtype=torch.bfloat16, device=x.device)
            plan.y_pairs = torch.zeros(P, H, dtype=torch.bfloat16, device=x.device)
        C.moe_plan(ids, wts, e_lo, E_local, bn, plan.counts, plan.offsets, plan.sorted_token, plan.sorted_pair,
                   plan.sorted_w, plan.tile_group, plan.tile_tok0, plan.tile_ntok, plan.meta)
        C.gather_rows(x, plan.sorted_token, plan.meta[1:2], plan.x_sorted[:P])
        x8, xs = fp8_quant_act(plan.x_sorted)
        C.wgemm_fp8(gu2, gu_s, x8, xs, plan.h_sorted, None, None, None, n_ff, True, n_ff, bn, 1, None, None, ws.status,
                    plan.tile_group, plan.tile_tok0, plan.tile_ntok, plan.meta, plan.max_tiles, 2 * n_ff, 0, None)
        h8, hs = fp8_quant_act(plan.h_sorted)
        C.wgemm_fp8(dn2, dn_s, h8, hs, plan.y_pairs, None, plan.sorted_w, plan.sorted_pair, H, False, 0, bn, 1, None,
                    None, ws.status, plan.tile_group, plan.tile_tok0, plan.tile_ntok, plan.meta, plan.max_tiles, H, 0,
                    None)
        y = plan.y_pairs
    if norm is None:
        C.moe_combine(y, ids, e_lo, e_lo + E_local, shared, shared_gate, residual, out, None, 0.0, 0.0, None)
        return out
    normed = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    C.moe_combine(y, ids, e_lo, e_lo + E_local, shared, shared_gate, residual, out, norm[0], norm[1], norm[2], normed)
    return out, normed


def token_logprobs(logits, chosen, n_top: int = 0):
    """(log-probability of chosen[r] in row r, top-n token ids [R, n], their log-probabilities [R, n])."""
    C = ext()
    R = logits.shape[0]
    lp = torch.empty(R, dtype=torch.float32, device=logits.device)
    ids = torch.empty(R, max(n_top, 1), dtype=torch.int32, device=logits.device)
    tl = torch.empty(R, max(n_top, 1), dtype=torch.float32, device=logits.device)
    C.token_logprobs(logits, chosen.int(), n_top, lp, ids, tl)
    return lp, ids[:, :n_top], tl[:, :n_top]


def spec_accept(target, cu, draft, n_draft):
    """Greedy acceptance on the device: (accepted drafts per sequence, the token after the accepted prefix,
    flag: some draft was rejected)."""
    C = ext()
    B = draft.shape[0]
    acc = torch.empty(B, dtype=torch.int32, device=target.device)
    bonus = torch.empty(B, dtype=torch.int32, device=target.device)
    rej = torch.zeros(1, dtype=torch.int32, device=target.device)
    C.spec_accept(target.int(), cu.int(), draft.int().contiguous(), n_draft.int(), acc, bonus, rej)
    return acc, bonus, rej


def argmax(logits, out=None, out_val=None):
    C = ext()
    rows, V = logits.shape
    ws = Workspace.get(logits.device)
    nblk = max(1, min(64, (V + 4095) // 4096))
    pv = ws.buf("argmax_v", (rows * nblk,), torch.float32)
    pi = ws.buf("argmax_i", (rows * nblk,), torch.int32)
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    C.argmax(logits, pv, pi, out, out_val)
    return out


def sample(logits, temperature, top_k, top_p, min_p, seeds, steps, out=None):
    C = ext()
    rows, V = logits.shape
    ws = Workspace.get(logits.device)
    scratch = ws.buf("sample", (rows * V,), torch.float32)
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    C.sample(logits, temperature, top_k, top_p, min_p, seeds, steps, scratch, out)
    return out


def causal_conv1d_silu(x, w, bias, conv_state, cu_seq, slots, write_state=True, out=None, max_len=None):
    """``max_len``: longest sequence of the step when known on the host; prompt-sized steps (>= 64 rows per
    sequence) run the token-parallel kernel."""
    C = ext()
    if out is None:
        out = torch.empty_like(x)
    T, n = x.shape[0], max(1, slots.numel())
    if max_len is None:
        max_len = T if T >= 64 * n else 0          # without the host figure: only clearly prompt-sized steps
    C.conv1d_silu(x, w, bias, conv_state, cu_seq, slots, out, write_state, int(max_len) if max_len >= 64 else 0)
    return out


def gdn_gates(a, b, A, dt_bias):
    C = ext()
    g = torch.empty(a.shape, dtype=torch.float32, device=a.device)
    beta = torch.empty_like(g)
    C.gdn_gates(a, b, A, dt_bias, g, beta)
    return g, beta


def gdn_chunk_plan(cu_host, device):
    """Host-side tables of the chunked scan for one step: 128-token blocks and per-sequence chunk ranges."""
    blk_t0, blk_n, seq_blk0, seq_nchunk, seq_t0, seq_len = [], [], [], [], [], []
    for i in range(len(cu_host) - 1):
        t0, n = cu_host[i], cu_host[i + 1] - cu_host[i]
        seq_blk0.append(len(blk_t0))
        seq_nchunk.append((n + 63) // 64)
        seq_t0.append(t0)
        seq_len.append(n)
        for b in range(0, n, 128):
            blk_t0.append(t0 + b)
            blk_n.append(min(128, n - b))
    i32 = dict(dtype=torch.int32, device=device)
    return tuple(torch.tensor(v, **i32) for v in (blk_t0, blk_n, seq_blk0, seq_nchunk, seq_t0, seq_len))


def gdn_chunked(qkv, g, beta, state, cu_host, slots, n_k, n_v, dk, dv, tiled_heads, scale, l2_eps=1e-6,
                write_state=True, out=None):
    """Gated delta rule over prompt-sized rows on the tensor cores (64-token chunks, ``csrc/gdn_chunk_sm100.cu``).
    ``cu_host``: the sequence boundaries as a Python list. Heads of 128 x 128 only."""
    C = ext()
    T = qkv.shape[0]
    ws = Workspace.get(qkv.device)
    blk_t0, blk_n, seq_blk0, seq_nchunk, seq_t0, seq_len = gdn_chunk_plan(cu_host, qkv.device)
    nb = int(blk_t0.numel())
    need = C.gdn_chunk_scratch_bytes(nb, n_v)
    scratch = ws._cache.get("gdn_chunk_scratch")
    if scratch is None or scratch.numel() < need:
        scratch = torch.empty(need, dtype=torch.uint8, device=qkv.device)
        ws._cache["gdn_chunk_scratch"] = scratch
    if out is None:
        out = torch.empty(T, n_v, dv, dtype=torch.bfloat16, device=qkv.device)
    C.gdn_chunk(qkv, g.contiguous(), beta.contiguous(), state, blk_t0, blk_n, seq_blk0, seq_nchunk, seq_t0, seq_len,
                slots, n_k, n_v, dk, dv, bool(tiled_heads), scale, l2_eps, out, bool(write_state), scratch, ws.status)
    return out


def gdn_recurrent(qkv, g, beta, state, cu_seq, slots, n_k, n_v, dk, dv, tiled_heads, scale, l2_eps=1e-6,
                  write_state=True, out=None, cu_host=None):
    C = ext()
    T = qkv.shape[0]
    # prompt chunks (many rows per sequence): the chunked tensor-core scan when the heads are 128 x 128, else the
    # column-per-thread kernel; decode rows run the state-streaming one
    prompt_rows = T >= 16 * max(1, slots.numel())
    if prompt_rows and dk == 128 and dv == 128 and T >= 64 and TUNE["gdn_chunk"] and qkv.stride(0) % 8 == 0:
        if cu_host is None:
            cu_host = cu_seq.tolist()
        return gdn_chunked(qkv, g, beta, state, cu_host, slots, n_k, n_v, dk, dv, tiled_heads, scale, l2_eps,
                           write_state, out)
    if out is None:
        out = torch.empty(T, n_v, dv, dtype=torch.bfloat16, device=qkv.device)
    C.gdn_recurrent(qkv, g, beta, state, cu_seq, slots, n_k, n_v, dk, dv, tiled_heads, scale, l2_eps, out,
                    write_state, True, prompt_rows)
    return out


def gdn_decode_fused_ok(n_k, n_v, dk, dv, conv_k) -> bool:
    return dk == dv and dk in (64, 128) and conv_k == 4 and n_k > 0 and n_v % n_k == 0 and n_v // n_k <= 4


def gdn_decode_fused(proj, conv_w, conv_state, A, dt_bias, norm_w, eps, act, state, slots, n_k, n_v, dk, dv,
                     tiled_heads, scale, l2_eps=1e-6, out=None):
    """One launch for the decode step of a Gated DeltaNet layer: conv + SiLU with history update, gates, delta rule
    with state update, gated RMS norm. ``proj`` [n_seqs, q|k|v|z|b|a] is the fused input projection of the step's
    tokens (one per sequence, in sequence order). Returns bf16 [n_seqs, n_v * dv]."""
    C = ext()
    n = slots.numel()
    if out is None:
        out = torch.empty(n, n_v * dv, dtype=torch.bfloat16, device=proj.device)
    C.gdn_decode_fused(proj, conv_w, conv_state, A, dt_bias, norm_w, eps, 0 if act == "silu" else 1, state, slots,
                       n_k, n_v, dk, dv, bool(tiled_heads), scale, l2_eps, out)
    return out


def mamba2_scan_ok(nh: int, hd: int, ng: int, ds: int) -> bool:
    """Head shapes the Mamba-2 kernel's thread layout covers (256 / hd threads per state row, <= 32 columns each)."""
    if hd <= 0 or hd > 256 or 256 % hd or hd & (hd - 1) or nh % max(ng, 1):
        return False
    W = 256 // hd
    return W <= 32 and ds % W == 0 and ds // W <= 32


def mamba2_scan(xbc, dt_raw, z, A, D, dt_bias, state, cu_seq, slots, nh, hd, ng, ds, write_state=True, out=None):
    """Mamba-2 recurrence over the step's tokens: xbc [T, nh*hd + 2*ng*ds] = x | B | C after the causal conv, dt_raw
    [T, nh], z [T, nh*hd] (bf16, row slices allowed), fp32 state [slots, nh, hd, ds] updated in place. Returns
    (S C + D x) * silu(z) as bf16 [T, nh*hd]."""
    C = ext()
    T = xbc.shape[0]
    if out is None:
        out = torch.empty(T, nh * hd, dtype=torch.bfloat16, device=xbc.device)
    if T == 0:
        return out
    C.mamba2_scan(xbc, dt_raw, z, A.float(), D.float(), dt_bias.float(), state, cu_seq, slots, nh, hd, ng, ds, out,
                  bool(write_state))
    return out


def gated_rmsnorm(o, z, w, eps, act="silu", out=None):
    C = ext()
    T, Hv, DV = o.shape
    if out is None:
        out = torch.empty_like(o)
    C.gated_rmsnorm(o, z, w, eps, Hv, DV, 0 if act == "silu" else 1, out)
    return out


def embed(ids, table, out=None):
    C = ext()
    if out is None:
        out = torch.empty(ids.numel(), table.shape[1], dtype=torch.bfloat16, device=table.device)
    C.embed(ids, table, out)
    return out
