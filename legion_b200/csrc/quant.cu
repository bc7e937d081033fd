// Block-scaled weight formats: NVFP4 (e2m1 codes, e4m3 scale per 16, fp32 tensor scale) and FP8 e4m3
// with 128x128 weight-block scales / 1x128 activation scales. Kernels here convert between these
// layouts and bf16 at load time and quantise activations; they also generate random weights on the
// device for benchmarks of models too large to initialise on the host.
//
// Counterparts in the reference: src/hf/nvfp4.rs (repack), src/cuda/fp8_mm.cu (fp8_quant,
// fp8_quant_dyn), src/cuda/sm120/nvfp4_a4.cu (nvfp4_a4_quant), src/cuda/dequant.cu.
#include "quant.h"

#include <cuda_fp8.h>

#include "common.cuh"

namespace lb {

__device__ __forceinline__ float e2m1_to_float(uint32_t c) {
  const float mag[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  const float v = mag[c & 7];
  return (c & 8) ? -v : v;
}
__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  __nv_fp8_e4m3 v;
  v.__x = b;
  return float(v);
}
__device__ __forceinline__ uint8_t float_to_e4m3(float f) {
  __nv_fp8_e4m3 v(f);
  return v.__x;
}
__device__ __forceinline__ uint32_t float_to_e2m1(float x) {
  // round to nearest representable magnitude, ties to the even code
  const float a = fabsf(x);
  uint32_t c;
  if (a <= 0.25f) c = 0;
  else if (a < 0.75f) c = 1;
  else if (a <= 1.25f) c = 2;
  else if (a < 1.75f) c = 3;
  else if (a <= 2.5f) c = 4;
  else if (a < 3.5f) c = 5;
  else if (a <= 5.f) c = 6;
  else c = 7;
  return c | (x < 0.f ? 8u : 0u);
}

// out[r, k] = e2m1(codes[r, k/2]) * e4m3(scales[r, k/16]) * global_scale ; one thread per byte pair.
__global__ void nvfp4_dequant_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                                     const float* __restrict__ global_scale, long rows, long K,
                                     __nv_bfloat16* __restrict__ out) {
  const long i = long(blockIdx.x) * blockDim.x + threadIdx.x;  // byte index
  if (i >= rows * (K / 2)) return;
  const long r = i / (K / 2);
  const long kb = i % (K / 2);
  const uint8_t b = codes[i];
  const float s = e4m3_to_float(scales[r * (K / 16) + (kb * 2) / 16]) * global_scale[0];
  const float lo = e2m1_to_float(b & 15) * s, hi = e2m1_to_float(b >> 4) * s;
  reinterpret_cast<__nv_bfloat162*>(out)[i] = __floats2bfloat162_rn(lo, hi);
}

int nvfp4_dequant_launch(const uint8_t* codes, const uint8_t* scales, const float* global_scale, long rows, long K,
                         void* out, cudaStream_t s) {
  if (K % 16) return 1;
  const long n = rows * (K / 2);
  if (n <= 0) return 0;
  nvfp4_dequant_kernel<<<unsigned((n + 255) / 256), 256, 0, s>>>(codes, scales, global_scale, rows, K,
                                                                 static_cast<__nv_bfloat16*>(out));
  return cudaGetLastError() != cudaSuccess;
}

// Quantise bf16 rows to NVFP4: per 16 elements scale = amax / 6 / global_scale rounded to e4m3.
// One thread per 16-element group.
__global__ void nvfp4_quant_kernel(const __nv_bfloat16* __restrict__ x, long ldx, const float* __restrict__ global_scale,
                                   long rows, long K, uint8_t* __restrict__ codes, uint8_t* __restrict__ scales) {
  const long i = long(blockIdx.x) * blockDim.x + threadIdx.x;
  const long groups = K / 16;
  if (i >= rows * groups) return;
  const long r = i / groups, g = i % groups;
  const __nv_bfloat16* p = x + r * ldx + g * 16;
  float v[16], amax = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    v[j] = __bfloat162float(p[j]);
    amax = fmaxf(amax, fabsf(v[j]));
  }
  const float gs = global_scale[0];
  const uint8_t sb = float_to_e4m3(amax / 6.f / gs);
  const float sdec = e4m3_to_float(sb) * gs;
  const float inv = sdec > 0.f ? 1.f / sdec : 0.f;
  scales[i] = sb;
  uint8_t* c = codes + r * (K / 2) + g * 8;
#pragma unroll
  for (int j = 0; j < 8; ++j) c[j] = uint8_t(float_to_e2m1(v[2 * j] * inv) | (float_to_e2m1(v[2 * j + 1] * inv) << 4));
}

int nvfp4_quant_launch(const void* x, long ldx, const float* global_scale, long rows, long K, uint8_t* codes,
                       uint8_t* scales, cudaStream_t s) {
  if (K % 16) return 1;
  const long n = rows * (K / 16);
  if (n <= 0) return 0;
  nvfp4_quant_kernel<<<unsigned((n + 255) / 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), ldx,
                                                               global_scale, rows, K, codes, scales);
  return cudaGetLastError() != cudaSuccess;
}

// out[r, k] = e4m3(w[r, k]) * scale[r / br, k / bk]
__global__ void fp8_block_dequant_kernel(const uint8_t* __restrict__ w, const float* __restrict__ scale, long rows,
                                         long K, int br, int bk, long scale_cols, __nv_bfloat16* __restrict__ out) {
  const long i = long(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows * K) return;
  const long r = i / K, k = i % K;
  out[i] = __float2bfloat16(e4m3_to_float(w[i]) * scale[(r / br) * scale_cols + k / bk]);
}

int fp8_block_dequant_launch(const uint8_t* w, const float* scale, long rows, long K, int br, int bk, void* out,
                             cudaStream_t s) {
  const long n = rows * K;
  if (n <= 0) return 0;
  const long scale_cols = (K + bk - 1) / bk;
  fp8_block_dequant_kernel<<<unsigned((n + 255) / 256), 256, 0, s>>>(w, scale, rows, K, br, bk, scale_cols,
                                                                     static_cast<__nv_bfloat16*>(out));
  return cudaGetLastError() != cudaSuccess;
}

// Block quantisation to e4m3: one CTA per (row block, k block); scale = amax / 448.
__global__ void fp8_block_quant_kernel(const __nv_bfloat16* __restrict__ x, long ldx, long rows, long K, int br, int bk,
                                       long scale_cols, uint8_t* __restrict__ out, float* __restrict__ scale) {
  const long rb = blockIdx.y, kb = blockIdx.x;
  __shared__ float red[8];
  __shared__ float s_scale;
  float amax = 0.f;
  const int n = br * bk;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const long r = rb * br + i / bk, k = kb * bk + i % bk;
    if (r < rows && k < K) amax = fmaxf(amax, fabsf(__bfloat162float(x[r * ldx + k])));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.f;
    for (int i = 0; i < int(blockDim.x / 32); ++i) m = fmaxf(m, red[i]);
    s_scale = m > 0.f ? m / 448.f : 1.f;
    scale[rb * scale_cols + kb] = s_scale;
  }
  __syncthreads();
  const float inv = 1.f / s_scale;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const long r = rb * br + i / bk, k = kb * bk + i % bk;
    if (r < rows && k < K) out[r * K + k] = float_to_e4m3(__bfloat162float(x[r * ldx + k]) * inv);
  }
}

int fp8_block_quant_launch(const void* x, long ldx, long rows, long K, int br, int bk, uint8_t* out, float* scale,
                           cudaStream_t s) {
  if (rows <= 0 || K <= 0) return 0;
  dim3 grid(unsigned((K + bk - 1) / bk), unsigned((rows + br - 1) / br));
  fp8_block_quant_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), ldx, rows, K, br, bk,
                                              (K + bk - 1) / bk, out, scale);
  return cudaGetLastError() != cudaSuccess;
}

// Activation quantisation to e4m3 with one fp32 scale per row and 128 columns: one warp per group (lane = 4
// consecutive elements, one 8-byte load and one 4-byte store), eight groups per CTA.
__global__ void __launch_bounds__(256)
fp8_act_quant_kernel(const __nv_bfloat16* __restrict__ x, long ldx, long rows, int groups_per_row,
                     uint8_t* __restrict__ out, float* __restrict__ scale) {
  const long g = long(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (g >= rows * groups_per_row) return;
  const int lane = threadIdx.x & 31;
  const long r = g / groups_per_row;
  const int kb = int(g % groups_per_row);
  const uint2 raw = *reinterpret_cast<const uint2*>(x + r * ldx + kb * 128 + lane * 4);
  const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  const float2 a = __bfloat1622float2(p0), b = __bfloat1622float2(p1);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float sc = amax > 0.f ? amax / 448.f : 1.f;
  const float inv = 1.f / sc;
  const uint32_t q = uint32_t(float_to_e4m3(a.x * inv)) | (uint32_t(float_to_e4m3(a.y * inv)) << 8) |
                     (uint32_t(float_to_e4m3(b.x * inv)) << 16) | (uint32_t(float_to_e4m3(b.y * inv)) << 24);
  *reinterpret_cast<uint32_t*>(out + r * (long(groups_per_row) * 128) + kb * 128 + lane * 4) = q;
  if (lane == 0) scale[g] = sc;
}

int fp8_act_quant_launch(const void* x, long ldx, long rows, long K, uint8_t* out, float* scale, cudaStream_t s) {
  if (rows <= 0 || K <= 0) return 0;
  if (K % 128 != 0 || ldx % 4 != 0 || (reinterpret_cast<uintptr_t>(x) & 7)) return 1;
  const long groups = rows * (K / 128);
  fp8_act_quant_kernel<<<unsigned((groups + 7) / 8), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), ldx, rows,
                                                                  int(K / 128), out, scale);
  return cudaGetLastError() != cudaSuccess;
}

// Deterministic N(0, std) weights from a counter-based generator (Box-Muller on two hashed words).
__device__ __forceinline__ uint32_t hash32(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdull; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ull; x ^= x >> 33;
  return uint32_t(x);
}
__global__ void randn_bf16_kernel(__nv_bfloat16* __restrict__ out, long n, float stdv, uint64_t seed) {
  for (long i = long(blockIdx.x) * blockDim.x + threadIdx.x; i < n / 2 + 1; i += long(gridDim.x) * blockDim.x) {
    const uint32_t a = hash32(seed * 0x9E3779B97F4A7C15ull + 2 * i), b = hash32(seed * 0x9E3779B97F4A7C15ull + 2 * i + 1);
    const float u1 = (float(a >> 8) + 1.f) * (1.f / 16777217.f), u2 = float(b >> 8) * (1.f / 16777216.f);
    const float rr = sqrtf(-2.f * __logf(u1)) * stdv;
    float sn, cs;
    __sincosf(6.283185307179586f * u2, &sn, &cs);
    if (2 * i < n) out[2 * i] = __float2bfloat16(rr * cs);
    if (2 * i + 1 < n) out[2 * i + 1] = __float2bfloat16(rr * sn);
  }
}

int randn_bf16_launch(void* out, long n, float stdv, uint64_t seed, cudaStream_t s) {
  if (n <= 0) return 0;
  randn_bf16_kernel<<<1184, 256, 0, s>>>(static_cast<__nv_bfloat16*>(out), n, stdv, seed);
  return cudaGetLastError() != cudaSuccess;
}

}  // namespace lb
