// GGUF block de-quantisation on the device: the raw tensor bytes are copied to the GPU as they sit in the file and
// expanded to bf16 there (one-time at load; the host no longer touches the weights element by element).
// One thread per 32 output elements; block layouts as written by ggml (Q8_0, Q4_0, Q4_K, Q5_K, Q6_K, IQ4_NL).
// Counterparts in the reference: src/cuda/dequant.cu and ggml's converters.
#include <cuda_fp16.h>

#include "common.cuh"
#include "quant.h"

namespace lb {

__device__ __forceinline__ float f16_at(const uint8_t* p) {
  return __half2float(__ushort_as_half(uint16_t(p[0]) | (uint16_t(p[1]) << 8)));
}
__device__ __forceinline__ void scale_min_k4(const uint8_t* sc, int j, float& d, float& m) {
  if (j < 4) {
    d = float(sc[j] & 63);
    m = float(sc[j + 4] & 63);
  } else {
    d = float((sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4));
    m = float((sc[j + 4] >> 4) | ((sc[j] >> 6) << 4));
  }
}
__constant__ float c_iq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

// type ids follow ggml: 2 Q4_0, 8 Q8_0, 12 Q4_K, 13 Q5_K, 14 Q6_K, 20 IQ4_NL
__global__ void gguf_dequant_kernel(const uint8_t* __restrict__ raw, int type, long n_groups,
                                    __nv_bfloat16* __restrict__ out) {
  const long g = long(blockIdx.x) * blockDim.x + threadIdx.x;   // group of 32 consecutive output elements
  if (g >= n_groups) return;
  __nv_bfloat16* o = out + g * 32;
  float v[32];
  if (type == 8) {
    const uint8_t* b = raw + g * 34;
    const float d = f16_at(b);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = float(int8_t(b[2 + i])) * d;
  } else if (type == 2 || type == 20) {
    const uint8_t* b = raw + g * 18;
    const float d = f16_at(b);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint8_t q = b[2 + i];
      if (type == 2) {
        v[i] = (float(q & 0xF) - 8.f) * d;
        v[i + 16] = (float(q >> 4) - 8.f) * d;
      } else {
        v[i] = c_iq4nl[q & 0xF] * d;
        v[i + 16] = c_iq4nl[q >> 4] * d;
      }
    }
  } else if (type == 12 || type == 13) {
    const int bb = type == 12 ? 144 : 176;
    const uint8_t* b = raw + (g >> 3) * bb;
    const int j = int(g & 7);                     // sub-block: 2i = low nibbles of chunk i, 2i+1 = high nibbles
    const float d = f16_at(b), dmin = f16_at(b + 2);
    float sc, mn;
    scale_min_k4(b + 4, j, sc, mn);
    const uint8_t* qs = b + (type == 12 ? 16 : 48) + (j >> 1) * 32;
    const uint8_t* qh = b + 16;                   // Q5_K only
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float q = (j & 1) ? float(qs[i] >> 4) : float(qs[i] & 0xF);
      if (type == 13) q += float((qh[i] >> j) & 1) * 16.f;
      v[i] = q * (d * sc) - dmin * mn;
    }
  } else if (type == 14) {
    const uint8_t* b = raw + (g >> 3) * 210;
    const int half = int(g & 7) >> 2, quarter = int(g & 3);    // 128-element half, 32-element quarter inside it
    const uint8_t* ql = b + half * 64;
    const uint8_t* qh = b + 128 + half * 32;
    const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192) + half * 8 + quarter * 2;
    const float d = f16_at(b + 208);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const uint8_t l = (quarter & 1) ? ql[32 + i] : ql[i];
      const int lo = (quarter & 2) ? (l >> 4) : (l & 0xF);
      const int hi = (qh[i] >> (2 * quarter)) & 3;
      v[i] = float(int8_t((lo | (hi << 4)) - 32)) * float(sc[i >> 4]) * d;
    }
  } else {
    return;
  }
#pragma unroll
  for (int i = 0; i < 32; i += 2)
    *reinterpret_cast<__nv_bfloat162*>(o + i) = __floats2bfloat162_rn(v[i], v[i + 1]);
}

int gguf_dequant_launch(const void* raw, int ggml_type, long n_elements, void* out_bf16, cudaStream_t s) {
  if (n_elements <= 0) return 0;
  const bool k_type = ggml_type == 12 || ggml_type == 13 || ggml_type == 14;
  if (!(k_type || ggml_type == 2 || ggml_type == 8 || ggml_type == 20)) return 1;
  if (n_elements % (k_type ? 256 : 32)) return 1;
  const long groups = n_elements / 32;
  gguf_dequant_kernel<<<unsigned((groups + 127) / 128), 128, 0, s>>>(static_cast<const uint8_t*>(raw), ggml_type,
                                                                      groups, static_cast<__nv_bfloat16*>(out_bf16));
  return cudaGetLastError() != cudaSuccess;
}

}  // namespace lb
