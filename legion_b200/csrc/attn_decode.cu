// Paged decode attention: flash-decoding over block tables with GQA head sharing.
//
// Grid (kv head x group tiles, sequence, split). Each CTA walks its share of the sequence's KV cells
// in chunks of 32 tokens per warp; the query heads that share the KV head are processed together so
// every K/V byte is read once per CTA. Per-warp online softmax, merged across the 4 warps at the end;
// each split writes (max, sum, unnormalised out) and attn_combine merges the splits. The number of
// splits is a launch constant and sequence lengths / block tables are data, so a captured CUDA graph
// stays valid as sequences grow.
//
// Counterpart in the reference: src/cuda/paged_attn/common.cuh (paged_decode, paged_combine).
#include "common.cuh"
#include "kernels.h"

namespace lb {

template <int D, int GT>
__global__ void __launch_bounds__(128) paged_decode_kernel(
    const __nv_bfloat16* __restrict__ q,  // [B, Hq, D]
    const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache, long cell_stride,
    const int* __restrict__ block_table, int table_width, int page, const int* __restrict__ ctx_lens, float scale,
    int window, int Hq, int Hkv, int n_splits, float* __restrict__ o_part, float* __restrict__ ml_part) {
  constexpr int LPT = 8;          // lanes per token in the QK phase
  constexpr int EPL = D / LPT;    // elements per lane in the QK phase
  constexpr int DPL = D / 32;     // output dims per lane in the PV phase
  const int G = Hq / Hkv;
  const int gtiles = (G + GT - 1) / GT;
  const int kvh = blockIdx.x / gtiles;
  const int g0 = (blockIdx.x % gtiles) * GT;
  const int gn = min(GT, G - g0);
  const int b = blockIdx.y;
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  __shared__ __align__(16) float q_s[GT][D];
  __shared__ __align__(16) float p_s[4][32][GT];     // [warp][token][g]
  __shared__ float m_s[4][GT], l_s[4][GT];
  __shared__ __align__(16) float o_s[4][GT][D];

  for (int i = threadIdx.x; i < GT * D; i += 128) {
    const int g = i / D, d = i % D;
    q_s[g][d] = (g < gn) ? __bfloat162float(q[(long(b) * Hq + kvh * G + g0 + g) * D + d]) * scale : 0.f;
  }
  __syncthreads();

  const int ctx = ctx_lens[b];
  const int start = (window > 0 && ctx > window) ? ctx - window : 0;
  // split the [start, ctx) range in units of 128 tokens
  const int n_units = (ctx - start + 127) / 128;
  const int units_per = (n_units + n_splits - 1) / n_splits;
  const int t_begin = start + split * units_per * 128;
  const int t_end = min(ctx, t_begin + units_per * 128);

  float m[GT], l[GT], acc[GT][DPL];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < DPL; ++j) acc[g][j] = 0.f;
  }
  const int* bt = block_table + long(b) * table_width;
  const int tg = lane / LPT;   // token within a quad
  const int tl = lane % LPT;   // lane within the token

  for (int c0 = t_begin + warp * 32; c0 < t_end; c0 += 128) {
    // ---- scores for 32 tokens, 4 per step; the K loads of QB steps are issued before any is used
    constexpr int QB = (D <= 128) ? 4 : 2;
#pragma unroll 1
    for (int q0 = 0; q0 < 8; q0 += QB) {
      uint4 kreg[QB][EPL / 8];
#pragma unroll
      for (int qi = 0; qi < QB; ++qi) {
        const int tok = c0 + (q0 + qi) * 4 + tg;
        if (tok < t_end) {
          const long cell = long(bt[tok / page]) * page + tok % page;
          const uint4* kp = reinterpret_cast<const uint4*>(k_cache + cell * cell_stride + long(kvh) * D + tl * EPL);
#pragma unroll
          for (int v8 = 0; v8 < EPL / 8; ++v8) kreg[qi][v8] = __ldg(&kp[v8]);
        } else {
#pragma unroll
          for (int v8 = 0; v8 < EPL / 8; ++v8) kreg[qi][v8] = make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int qi = 0; qi < QB; ++qi) {
        const int qd = q0 + qi;
        const int tok = c0 + qd * 4 + tg;
        float s[GT];
#pragma unroll
        for (int g = 0; g < GT; ++g) s[g] = 0.f;
#pragma unroll
        for (int v8 = 0; v8 < EPL / 8; ++v8) {
          const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kreg[qi][v8]);
          float kf[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(k2[j]);
            kf[2 * j] = f.x;
            kf[2 * j + 1] = f.y;
          }
#pragma unroll
          for (int g = 0; g < GT; ++g) {
            const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][tl * EPL + v8 * 8]);
            const float4 qb = *reinterpret_cast<const float4*>(&q_s[g][tl * EPL + v8 * 8 + 4]);
            s[g] += qa.x * kf[0] + qa.y * kf[1] + qa.z * kf[2] + qa.w * kf[3] + qb.x * kf[4] + qb.y * kf[5] +
                    qb.z * kf[6] + qb.w * kf[7];
          }
        }
#pragma unroll
        for (int g = 0; g < GT; ++g) {
          s[g] += __shfl_xor_sync(0xffffffffu, s[g], 1);
          s[g] += __shfl_xor_sync(0xffffffffu, s[g], 2);
          s[g] += __shfl_xor_sync(0xffffffffu, s[g], 4);
        }
        if (tl == 0) {
#pragma unroll
          for (int g = 0; g < GT; ++g) p_s[warp][qd * 4 + tg][g] = (tok < t_end) ? s[g] : -INFINITY;
        }
      }
    }
    __syncwarp();
    // ---- online softmax over the 32 tokens (lane = token)
    float alpha[GT];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      const float sv = p_s[warp][lane][g];
      float mx = sv;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float mn = fmaxf(m[g], mx);
      const float p = (sv == -INFINITY) ? 0.f : __expf(sv - mn);
      float ps = p;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
      alpha[g] = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - mn);
      l[g] = l[g] * alpha[g] + ps;
      m[g] = mn;
      p_s[warp][lane][g] = p;
    }
    __syncwarp();
#pragma unroll
    for (int g = 0; g < GT; ++g)
#pragma unroll
      for (int j = 0; j < DPL; ++j) acc[g][j] *= alpha[g];
    // ---- PV: lane owns DPL output dims
    const int nt = min(32, t_end - c0);
#pragma unroll 8
    for (int t = 0; t < nt; ++t) {
      const int tok = c0 + t;
      const long cell = long(bt[tok / page]) * page + tok % page;
      const __nv_bfloat16* vp = v_cache + cell * cell_stride + long(kvh) * D + lane * DPL;
      float vf[DPL];
      if constexpr (DPL == 2) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vp));
        vf[0] = f.x; vf[1] = f.y;
      } else if constexpr (DPL == 4) {
        const uint2 u = *reinterpret_cast<const uint2*>(vp);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
        const float2 f0 = __bfloat1622float2(u2[0]), f1 = __bfloat1622float2(u2[1]);
        vf[0] = f0.x; vf[1] = f0.y; vf[2] = f1.x; vf[3] = f1.y;
      } else {
        const uint4 u = *reinterpret_cast<const uint4*>(vp);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(u2[j]);
          vf[2 * j] = f.x;
          vf[2 * j + 1] = f.y;
        }
      }
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        const float p = p_s[warp][t][g];
#pragma unroll
        for (int j = 0; j < DPL; ++j) acc[g][j] += p * vf[j];
      }
    }
    __syncwarp();
  }

  // ---- merge the 4 warps
  if (lane == 0) {
#pragma unroll
    for (int g = 0; g < GT; ++g) { m_s[warp][g] = m[g]; l_s[warp][g] = l[g]; }
  }
#pragma unroll
  for (int g = 0; g < GT; ++g)
#pragma unroll
    for (int j = 0; j < DPL; ++j) o_s[warp][g][lane * DPL + j] = acc[g][j];
  __syncthreads();
  for (int i = threadIdx.x; i < gn * D; i += 128) {
    const int g = i / D, d = i % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, m_s[w][g]);
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float a = (m_s[w][g] == -INFINITY) ? 0.f : __expf(m_s[w][g] - mm);
      ll += l_s[w][g] * a;
      oo += o_s[w][g][d] * a;
    }
    const long row = (long(b) * Hq + kvh * G + g0 + g) * n_splits + split;
    o_part[row * D + d] = oo;
    if (d == 0) {
      ml_part[row * 2] = mm;
      ml_part[row * 2 + 1] = ll;
    }
  }
}

// out[b, h, :] = sum_s o_part * exp(m_s - M) / sum_s l_s * exp(m_s - M)
__global__ void attn_combine_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part, int n_splits,
                                    int D, __nv_bfloat16* __restrict__ out) {
  const long row = blockIdx.x;  // b * Hq + h
  float mm = -INFINITY;
  for (int s = 0; s < n_splits; ++s) mm = fmaxf(mm, ml_part[(row * n_splits + s) * 2]);
  float ll = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float m = ml_part[(row * n_splits + s) * 2];
    if (m != -INFINITY) ll += ml_part[(row * n_splits + s) * 2 + 1] * __expf(m - mm);
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float m = ml_part[(row * n_splits + s) * 2];
      if (m != -INFINITY) o += o_part[(row * n_splits + s) * D + d] * __expf(m - mm);
    }
    out[row * D + d] = __float2bfloat16(ll > 0.f ? o / ll : 0.f);
  }
}

int attn_combine_launch(const float* o_part, const float* ml_part, int n_splits, int rows, int D, void* out,
                        cudaStream_t s) {
  attn_combine_kernel<<<rows, D < 128 ? D : 128, 0, s>>>(o_part, ml_part, n_splits, D,
                                                         static_cast<__nv_bfloat16*>(out));
  return cudaGetLastError() != cudaSuccess ? 1 : 0;
}

int paged_decode_launch(const void* q, const void* k_cache, const void* v_cache, long cell_stride,
                        const int* block_table, int table_width, int page, const int* ctx_lens, float scale, int window,
                        int B, int Hq, int Hkv, int D, int n_splits, float* o_part, float* ml_part, void* out,
                        cudaStream_t s) {
  if (B <= 0) return 0;
  if (Hq % Hkv) return 1;
  const int G = Hq / Hkv;
  int GT = G >= 8 ? 8 : (G > 2 ? 4 : (G == 2 ? 2 : 1));
  const int gtiles = (G + GT - 1) / GT;
  dim3 grid(Hkv * gtiles, B, n_splits);
#define LB_CASE(DD, GG)                                                                                         \
  if (D == DD && GT == GG) {                                                                                    \
    paged_decode_kernel<DD, GG><<<grid, 128, 0, s>>>(                                                           \
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_cache),                       \
        static_cast<const __nv_bfloat16*>(v_cache), cell_stride, block_table, table_width, page, ctx_lens,      \
        scale, window, Hq, Hkv, n_splits, o_part, ml_part);                                                     \
  } else
  LB_CASE(64, 1) LB_CASE(64, 2) LB_CASE(64, 4) LB_CASE(64, 8)
  LB_CASE(128, 1) LB_CASE(128, 2) LB_CASE(128, 4) LB_CASE(128, 8)
  LB_CASE(256, 1) LB_CASE(256, 2) LB_CASE(256, 4) LB_CASE(256, 8)
  { return 1; }
#undef LB_CASE
  if (cudaGetLastError() != cudaSuccess) return 2;
  attn_combine_kernel<<<B * Hq, D < 128 ? D : 128, 0, s>>>(o_part, ml_part, n_splits, D,
                                                           static_cast<__nv_bfloat16*>(out));
  return cudaGetLastError() != cudaSuccess ? 2 : 0;
}

}  // namespace lb
