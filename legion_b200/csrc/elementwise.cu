// Row-wise fused kernels: RMSNorm (+residual add), per-head QK norm + RoPE + paged KV append,
// sigmoid output gate, SwiGLU, embedding gather. All bf16 in / bf16 out with fp32 math.
//
// Counterparts in the reference: src/cuda/norm_rope.cu (norm_rope_kernel, kv_append_kernel),
// src/cuda/fused.cu (rms_norm_bf16, gate_bf16).
#include "common.cuh"
#include "kernels.h"

namespace lb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < THREADS / 32) ? red[l] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// y = rmsnorm(x (+ residual)) * w ; optionally writes the sum back as the new residual stream.
// One CTA per row; H must be a multiple of 8 (16-byte vectors).
__global__ void __launch_bounds__(256) rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, long ldx,
                                                      const __nv_bfloat16* __restrict__ res_in, long ldri,
                                                      __nv_bfloat16* __restrict__ res_out, long ldro,
                                                      const float* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                                      long ldy, int H, float eps, float w_offset) {
  __shared__ float red[8];
  griddep_wait();
  griddep_launch();
  const long row = blockIdx.x;
  const uint4* xv = reinterpret_cast<const uint4*>(x + row * ldx);
  const uint4* rv = res_in ? reinterpret_cast<const uint4*>(res_in + row * ldri) : nullptr;
  uint4* ro = res_out ? reinterpret_cast<uint4*>(res_out + row * ldro) : nullptr;
  const int nv = H / 8;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nv; i += 256) {
    uint4 a = xv[i];
    __nv_bfloat162* ap = reinterpret_cast<__nv_bfloat162*>(&a);
    if (rv) {
      uint4 b = rv[i];
      __nv_bfloat162* bp = reinterpret_cast<__nv_bfloat162*>(&b);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 fa = __bfloat1622float2(ap[j]), fb = __bfloat1622float2(bp[j]);
        ap[j] = __floats2bfloat162_rn(fa.x + fb.x, fa.y + fb.y);
      }
    }
    if (ro) ro[i] = a;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(ap[j]);
      ss += f.x * f.x + f.y * f.y;
    }
  }
  ss = block_sum<256>(ss, red);
  const float inv = rsqrtf(ss / float(H) + eps);
  uint4* yv = reinterpret_cast<uint4*>(y + row * ldy);
  for (int i = threadIdx.x; i < nv; i += 256) {
    uint4 a;
    if (ro) {
      a = ro[i];
    } else {
      a = xv[i];
      if (rv) {  // recompute the sum when it was not stored
        uint4 b = rv[i];
        __nv_bfloat162* ap = reinterpret_cast<__nv_bfloat162*>(&a);
        __nv_bfloat162* bp = reinterpret_cast<__nv_bfloat162*>(&b);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 fa = __bfloat1622float2(ap[j]), fb = __bfloat1622float2(bp[j]);
          ap[j] = __floats2bfloat162_rn(fa.x + fb.x, fa.y + fb.y);
        }
      }
    }
    __nv_bfloat162* ap = reinterpret_cast<__nv_bfloat162*>(&a);
    const float4 w0 = reinterpret_cast<const float4*>(w)[2 * i];
    const float4 w1 = reinterpret_cast<const float4*>(w)[2 * i + 1];
    const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(ap[j]);
      ap[j] = __floats2bfloat162_rn(f.x * inv * (ww[2 * j] + w_offset), f.y * inv * (ww[2 * j + 1] + w_offset));
    }
    yv[i] = a;
  }
}

int rmsnorm_launch(const void* x, long ldx, const void* res_in, long ldri, void* res_out, long ldro, const float* w,
                   void* y, long ldy, int rows, int H, float eps, float w_offset, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (H % 8) return 1;
  return launch_pdl(rmsnorm_kernel, dim3(rows), dim3(256), 0, s, static_cast<const __nv_bfloat16*>(x), ldx,
                    static_cast<const __nv_bfloat16*>(res_in), ldri, static_cast<__nv_bfloat16*>(res_out), ldro, w,
                    static_cast<__nv_bfloat16*>(y), ldy, H, eps, w_offset) != cudaSuccess;
}

// One warp per (token, head). Heads 0..Hq-1 are queries, then Hkv keys, then Hkv values, read from
// the fused QKV projection output. Queries: optional RMS norm over the head, RoPE (rotate-half
// pairing (i, i + rot/2), rot % 64 == 0), written to q_out. Keys: norm + RoPE, written into the paged
// cache cell slot[t]. Values: copied into the cache. q heads may be laid out [q | gate] (stride 2D).
template <int D>
__global__ void __launch_bounds__(128) qk_norm_rope_append_kernel(
    const __nv_bfloat16* __restrict__ qkv, long ld_qkv, int q_head_stride, int k_off, int v_off,
    const float* __restrict__ qw, const float* __restrict__ kw, float eps, float w_offset,
    const float* __restrict__ cos_sin, int rot, const int* __restrict__ positions, const long* __restrict__ slots,
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
    long cache_cell_stride, int T, int Hq, int Hkv) {
  constexpr int N = D / 32;
  griddep_wait();
  griddep_launch();
  const int lane = threadIdx.x & 31;
  const long gw = (long(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int heads = Hq + 2 * Hkv;
  if (gw >= long(T) * heads) return;
  const int t = int(gw / heads);
  const int h = int(gw % heads);
  const __nv_bfloat16* src;
  const float* nw = nullptr;
  int kind;  // 0 q, 1 k, 2 v
  if (h < Hq) {
    kind = 0; src = qkv + t * ld_qkv + long(h) * q_head_stride; nw = qw;
  } else if (h < Hq + Hkv) {
    kind = 1; src = qkv + t * ld_qkv + k_off + long(h - Hq) * D; nw = kw;
  } else {
    kind = 2; src = qkv + t * ld_qkv + v_off + long(h - Hq - Hkv) * D;
  }
  float v[N];
#pragma unroll
  for (int j = 0; j < N; ++j) v[j] = __bfloat162float(src[lane + 32 * j]);
  if (kind != 2) {
    if (nw) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < N; ++j) ss += v[j] * v[j];
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / float(D) + eps);
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = v[j] * inv * (nw[lane + 32 * j] + w_offset);
    }
    if (rot > 0) {
      const int half = rot / 2;
      const int hj = half / 32;  // partner register offset
      const float* cs = cos_sin + long(positions[t]) * rot;  // [cos(half) | sin(half)]
#pragma unroll
      for (int j = 0; j < N; ++j) {
        if (j < hj) {
          const int i = lane + 32 * j;
          const float c = cs[i], s = cs[half + i];
          const float a = v[j], b = v[j + hj];
          v[j] = a * c - b * s;
          v[j + hj] = b * c + a * s;
        }
      }
    }
  }
  __nv_bfloat16* dst;
  if (kind == 0) {
    dst = q_out + (long(t) * Hq + h) * D;
  } else {
    const long cell = slots[t];
    if (cell < 0) return;
    __nv_bfloat16* base = (kind == 1) ? k_cache : v_cache;
    const int hk = (kind == 1) ? h - Hq : h - Hq - Hkv;
    dst = base + cell * cache_cell_stride + long(hk) * D;
  }
#pragma unroll
  for (int j = 0; j < N; ++j) dst[lane + 32 * j] = __float2bfloat16(v[j]);
}

int qk_norm_rope_append_launch(const void* qkv, long ld_qkv, int q_head_stride, int k_off, int v_off, const float* qw,
                               const float* kw, float eps, float w_offset, const float* cos_sin, int rot,
                               const int* positions, const long* slots, void* q_out, void* k_cache, void* v_cache,
                               long cache_cell_stride, int T, int Hq, int Hkv, int D, cudaStream_t s) {
  if (T <= 0) return 0;
  if (rot % 64 != 0 || rot > D) return 1;
  const long warps = long(T) * (Hq + 2 * Hkv);
  const int blocks = int((warps * 32 + 127) / 128);
#define LB_D(DD)                                                                                                   \
  if (D == DD) {                                                                                                   \
    return launch_pdl(qk_norm_rope_append_kernel<DD>, dim3(blocks), dim3(128), 0, s,                              \
                      static_cast<const __nv_bfloat16*>(qkv), ld_qkv, q_head_stride, k_off, v_off, qw, kw, eps,    \
                      w_offset, cos_sin, rot, positions, slots, static_cast<__nv_bfloat16*>(q_out),                \
                      static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache),                  \
                      cache_cell_stride, T, Hq, Hkv) != cudaSuccess;                                               \
  }
  LB_D(64) LB_D(128) LB_D(256)
#undef LB_D
  return 1;
}

// out[t, h, :] = attn[t, h, :] * sigmoid(gate[t, h, :]) where gate sits in the Q projection output
// at column h * q_head_stride + D.
__global__ void sigmoid_gate_kernel(const __nv_bfloat16* __restrict__ attn, const __nv_bfloat16* __restrict__ qkv,
                                    long ld_qkv, int q_head_stride, int D, int Hq, __nv_bfloat16* __restrict__ out,
                                    long n) {
  const long i = long(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int d = int(i % D);
  const long th = i / D;
  const int h = int(th % Hq);
  const long t = th / Hq;
  const float g = __bfloat162float(qkv[t * ld_qkv + long(h) * q_head_stride + D + d]);
  const float a = __bfloat162float(attn[i]);
  out[i] = __float2bfloat16(a / (1.f + __expf(-g)));
}

int sigmoid_gate_launch(const void* attn, const void* qkv, long ld_qkv, int q_head_stride, int D, int Hq, void* out,
                        long T, cudaStream_t s) {
  const long n = T * Hq * D;
  if (n <= 0) return 0;
  sigmoid_gate_kernel<<<int((n + 255) / 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(attn),
                                                           static_cast<const __nv_bfloat16*>(qkv), ld_qkv,
                                                           q_head_stride, D, Hq, static_cast<__nv_bfloat16*>(out), n);
  return cudaGetLastError() != cudaSuccess;
}

// out[t, :F] = silu(x[t, :F]) * x[t, F:2F]   (act = 0) ; gelu-tanh gate (act = 1) ; relu^2 of x[:F] alone (act = 2)
__global__ void glu_kernel(const __nv_bfloat16* __restrict__ x, long ldx, __nv_bfloat16* __restrict__ out, long ldo,
                           int F, long n, int act) {
  const long i = long(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long t = i / F;
  const int f = int(i % F);
  const float g = __bfloat162float(x[t * ldx + f]);
  float r;
  if (act == 2) {
    const float m = fmaxf(g, 0.f);
    r = m * m;
  } else {
    const float u = __bfloat162float(x[t * ldx + F + f]);
    if (act == 0) {
      r = g / (1.f + __expf(-g)) * u;
    } else {
      const float c = 0.7978845608028654f * (g + 0.044715f * g * g * g);
      r = 0.5f * g * (1.f + tanhf(c)) * u;
    }
  }
  out[t * ldo + f] = __float2bfloat16(r);
}

int glu_launch(const void* x, long ldx, void* out, long ldo, int F, long T, int act, cudaStream_t s) {
  const long n = T * F;
  if (n <= 0) return 0;
  glu_kernel<<<int((n + 255) / 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), ldx,
                                                  static_cast<__nv_bfloat16*>(out), ldo, F, n, act);
  return cudaGetLastError() != cudaSuccess;
}

// out[t, :] = table[ids[t], :]  (16-byte vectors; H % 8 == 0)
__global__ void embed_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table, long ldt,
                             __nv_bfloat16* __restrict__ out, long ldo, int H, int vocab) {
  const long t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const uint4* src = reinterpret_cast<const uint4*>(table + long(id) * ldt);
  uint4* dst = reinterpret_cast<uint4*>(out + t * ldo);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

int embed_launch(const int* ids, const void* table, long ldt, void* out, long ldo, int T, int H, int vocab,
                 cudaStream_t s) {
  if (T <= 0) return 0;
  if (H % 8) return 1;
  embed_kernel<<<T, 128, 0, s>>>(ids, static_cast<const __nv_bfloat16*>(table), ldt,
                                 static_cast<__nv_bfloat16*>(out), ldo, H, vocab);
  return cudaGetLastError() != cudaSuccess;
}

}  // namespace lb
