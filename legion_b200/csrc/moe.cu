// MoE routing: top-k selection, the expert-major routing plan that drives the grouped GEMM, row
// gather into expert order, and the weighted combine back to token order.
//
// The plan is deterministic: pairs of one expert keep their (token, choice) order, so the grouped
// GEMM and the combine give the same bits run to run.
//
// Counterparts in the reference: src/cuda/fused.cu (router_topk, router_weights, moe_combine,
// shexp_gate), src/cuda/moe_gemm.cu (prep, plan, scatter, reduce).
#include "common.cuh"
#include "ep.h"
#include "kernels.h"

namespace lb {

// One warp per token. mode 0: softmax over all experts -> top-k -> renormalise (optional).
// mode 1: sigmoid scores, selection by score + bias, optional group-limited routing (n_group groups,
// keep topk_group groups ranked by the sum of their two best biased scores), weights = unbiased
// scores of the chosen experts, renormalised and multiplied by route_scale.
template <int MAXE>
__global__ void __launch_bounds__(128) router_topk_kernel(const float* __restrict__ logits, long ldl,
                                                          const float* __restrict__ bias, int E, int k, int mode,
                                                          int renorm, float route_scale, int n_group, int topk_group,
                                                          int* __restrict__ ids, float* __restrict__ wts, int T) {
  constexpr int PER = MAXE / 32;
  const int lane = threadIdx.x & 31;
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (t >= T) return;
  float sc[PER], sel[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = lane + 32 * j;
    sc[j] = (e < E) ? logits[t * ldl + e] : -INFINITY;
    mx = fmaxf(mx, sc[j]);
  }
  if (mode == 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      sc[j] = (lane + 32 * j < E) ? __expf(sc[j] - mx) : 0.f;
      sum += sc[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      sc[j] *= inv;
      sel[j] = (lane + 32 * j < E) ? sc[j] : -INFINITY;
    }
  } else {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = lane + 32 * j;
      if (e < E) {
        sc[j] = 1.f / (1.f + __expf(-sc[j]));
        sel[j] = sc[j] + (bias ? bias[e] : 0.f);
      } else {
        sc[j] = 0.f;
        sel[j] = -INFINITY;
      }
    }
    if (n_group > 1 && topk_group < n_group) {
      // group score = sum of the two best biased scores in the group; groups are contiguous ranges.
      const int gs = E / n_group;
      float keep_thresh_rank[1];
      (void)keep_thresh_rank;
      // every lane computes all group scores through shared shuffles: loop groups (n_group <= 32)
      float my_gscore = -INFINITY;  // lane g holds the score of group g
      for (int g = 0; g < n_group; ++g) {
        float b1 = -INFINITY, b2 = -INFINITY;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
          const int e = lane + 32 * j;
          if (e < E && e / gs == g) {
            const float v = sel[j];
            if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
          }
        }
        // merge (b1, b2) across lanes
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float o1 = __shfl_xor_sync(0xffffffffu, b1, o);
          const float o2 = __shfl_xor_sync(0xffffffffu, b2, o);
          const float n1 = fmaxf(b1, o1);
          const float n2 = fmaxf(fminf(b1, o1), fmaxf(b2, o2));
          b1 = n1; b2 = n2;
        }
        if (lane == g) my_gscore = b1 + (b2 == -INFINITY ? 0.f : b2);
      }
      // rank of each group = number of groups with a better score (ties: lower index wins)
      int rank = 0;
      for (int g = 0; g < n_group; ++g) {
        const float og = __shfl_sync(0xffffffffu, my_gscore, g);
        if (lane < n_group && (og > my_gscore || (og == my_gscore && g < lane))) ++rank;
      }
      const unsigned keep_mask = __ballot_sync(0xffffffffu, lane < n_group && rank < topk_group);
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int e = lane + 32 * j;
        if (e < E && !((keep_mask >> (e / gs)) & 1u)) sel[j] = -INFINITY;
      }
    }
  }
  // iterative arg-max, ties to the lower expert index
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int i = 0; i < k; ++i) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = lane + 32 * j;
      if (sel[j] > bv) { bv = sel[j]; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
    }
    // fetch the unbiased score of the winner
    float w = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      if (lane + 32 * j == be) { w = sc[j]; sel[j] = -INFINITY; }
    }
    w = __shfl_sync(0xffffffffu, w, be & 31);
    wsum += w;
    if (lane == i) { my_w = w; my_id = be; }
  }
  if (lane < k) {
    float w = my_w;
    if (renorm) w = w / fmaxf(wsum, 6.1e-5f);
    ids[t * k + lane] = my_id;
    wts[t * k + lane] = w * route_scale;
  }
}

int router_topk_launch(const float* logits, long ldl, const float* bias, int E, int k, int mode, int renorm,
                       float route_scale, int n_group, int topk_group, int* ids, float* wts, int T, cudaStream_t s) {
  if (T <= 0) return 0;
  if (k > 32 || E > 512 || n_group > 32) return 1;
  const int blocks = (T * 32 + 127) / 128;
  if (E <= 128)
    router_topk_kernel<128><<<blocks, 128, 0, s>>>(logits, ldl, bias, E, k, mode, renorm, route_scale, n_group,
                                                   topk_group, ids, wts, T);
  else if (E <= 256)
    router_topk_kernel<256><<<blocks, 128, 0, s>>>(logits, ldl, bias, E, k, mode, renorm, route_scale, n_group,
                                                   topk_group, ids, wts, T);
  else
    router_topk_kernel<512><<<blocks, 128, 0, s>>>(logits, ldl, bias, E, k, mode, renorm, route_scale, n_group,
                                                   topk_group, ids, wts, T);
  return cudaGetLastError() != cudaSuccess;
}

// ---------------------------------------------------------------------------------------------
// routing plan
// ---------------------------------------------------------------------------------------------
// pass 1: one CTA per local expert counts its pairs.
__global__ void __launch_bounds__(256) moe_count_kernel(const int* __restrict__ ids, int n_pairs, int e_lo,
                                                        int* __restrict__ counts) {
  const int e = e_lo + blockIdx.x;
  int c = 0;
  for (int p = threadIdx.x; p < n_pairs; p += 256) c += (ids[p] == e);
  __shared__ int red[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int i = 0; i < 8; ++i) t += red[i];
    counts[blockIdx.x] = t;
  }
}
// pass 2: one CTA scans the counts: row offsets per expert and the token-tile list (tile = up to bn
// consecutive sorted rows of one expert). meta = {n_tiles, n_rows}.
__global__ void __launch_bounds__(512) moe_scan_kernel(const int* __restrict__ counts, int n_local, int bn,
                                                       int* __restrict__ offsets, int* __restrict__ tile_group,
                                                       int* __restrict__ tile_tok0, int* __restrict__ tile_ntok,
                                                       int max_tiles, int* __restrict__ meta) {
  __shared__ int s_cnt[512], s_off[513], s_toff[513];
  const int e = threadIdx.x;
  s_cnt[e] = (e < n_local) ? counts[e] : 0;
  __syncthreads();
  if (e == 0) {
    int o = 0, to = 0;
    for (int i = 0; i < n_local; ++i) {
      s_off[i] = o;
      s_toff[i] = to;
      o += s_cnt[i];
      to += (s_cnt[i] + bn - 1) / bn;
    }
    s_off[n_local] = o;
    s_toff[n_local] = to;
    meta[0] = to < max_tiles ? to : max_tiles;
    meta[1] = o;
  }
  __syncthreads();
  if (e < n_local) {
    offsets[e] = s_off[e];
    const int nt = (s_cnt[e] + bn - 1) / bn;
    for (int i = 0; i < nt; ++i) {
      const int ti = s_toff[e] + i;
      if (ti < max_tiles) {
        tile_group[ti] = e;
        tile_tok0[ti] = s_off[e] + i * bn;
        tile_ntok[ti] = min(bn, s_cnt[e] - i * bn);
      }
    }
  }
  if (e == 0) offsets[n_local] = s_off[n_local];
}
// pass 3: one CTA per local expert writes its pairs, in pair order, at its offset.
__global__ void __launch_bounds__(256) moe_fill_kernel(const int* __restrict__ ids, const float* __restrict__ wts,
                                                       int n_pairs, int k, int e_lo, const int* __restrict__ offsets,
                                                       int* __restrict__ sorted_token, int* __restrict__ sorted_pair,
                                                       float* __restrict__ sorted_w) {
  const int e = e_lo + blockIdx.x;
  const int base0 = offsets[blockIdx.x];
  __shared__ int warp_tot[8];
  __shared__ int running;
  if (threadIdx.x == 0) running = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int p0 = 0; p0 < n_pairs; p0 += 256) {
    const int p = p0 + threadIdx.x;
    const bool hit = p < n_pairs && ids[p] == e;
    const unsigned bal = __ballot_sync(0xffffffffu, hit);
    const int before = __popc(bal & ((1u << lane) - 1));
    if (lane == 0) warp_tot[warp] = __popc(bal);
    __syncthreads();
    int wbase = 0;
    for (int w = 0; w < warp; ++w) wbase += warp_tot[w];
    const int base = running;
    if (hit) {
      const int dst = base0 + base + wbase + before;
      sorted_token[dst] = p / k;
      sorted_pair[dst] = p;
      sorted_w[dst] = wts[p];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int t = 0;
      for (int w = 0; w < 8; ++w) t += warp_tot[w];
      running = base + t;
    }
    __syncthreads();
  }
}

int moe_plan_launch(const int* ids, const float* wts, int n_tokens, int k, int e_lo, int n_local, int bn, int* counts,
                    int* offsets, int* sorted_token, int* sorted_pair, float* sorted_w, int* tile_group,
                    int* tile_tok0, int* tile_ntok, int max_tiles, int* meta, cudaStream_t s) {
  if (n_local <= 0 || n_local > 512) return 1;
  const int n_pairs = n_tokens * k;
  moe_count_kernel<<<n_local, 256, 0, s>>>(ids, n_pairs, e_lo, counts);
  moe_scan_kernel<<<1, 512, 0, s>>>(counts, n_local, bn, offsets, tile_group, tile_tok0, tile_ntok, max_tiles, meta);
  moe_fill_kernel<<<n_local, 256, 0, s>>>(ids, wts, n_pairs, k, e_lo, offsets, sorted_token, sorted_pair, sorted_w);
  return cudaGetLastError() != cudaSuccess;
}

int moe_tiles_launch(const int* counts, int n_local, int bn, int* offsets, int* tile_group, int* tile_tok0,
                     int* tile_ntok, int max_tiles, int* meta, cudaStream_t s) {
  if (n_local <= 0 || n_local > 512) return 1;
  moe_scan_kernel<<<1, 512, 0, s>>>(counts, n_local, bn, offsets, tile_group, tile_tok0, tile_ntok, max_tiles, meta);
  return cudaGetLastError() != cudaSuccess;
}

// dst[i, :] = src[rows[i], :] for i < *n_rows (device scalar); 16-byte vectors.
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ src, long lds, const int* __restrict__ rows,
                                   const int* __restrict__ n_rows, __nv_bfloat16* __restrict__ dst, long ldd, int H) {
  const int n = *n_rows;
  for (int i = blockIdx.x; i < n; i += gridDim.x) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src + long(rows[i]) * lds);
    uint4* d4 = reinterpret_cast<uint4*>(dst + long(i) * ldd);
    for (int j = threadIdx.x; j < H / 8; j += blockDim.x) d4[j] = s4[j];
  }
}

int gather_rows_launch(const void* src, long lds, const int* rows, const int* n_rows, void* dst, long ldd, int H,
                       int max_rows, cudaStream_t s) {
  if (max_rows <= 0) return 0;
  if (H % 8) return 1;
  const int grid = max_rows < 4096 ? max_rows : 4096;
  gather_rows_kernel<<<grid, 128, 0, s>>>(static_cast<const __nv_bfloat16*>(src), lds, rows, n_rows,
                                          static_cast<__nv_bfloat16*>(dst), ldd, H);
  return cudaGetLastError() != cudaSuccess;
}

// out[t, :] = (residual[t, :]) + sum_j y[t*k + j, :] (rows whose expert is outside [e_lo, e_hi) are skipped)
//             + shared[t, :] * (shared_gate ? sigmoid(shared_gate[t]) : 1)
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, long ldy, const int* __restrict__ ids, int k,
                                   int e_lo, int e_hi, const __nv_bfloat16* __restrict__ shared, long lds,
                                   const float* __restrict__ shared_gate, const __nv_bfloat16* __restrict__ residual,
                                   long ldr, __nv_bfloat16* __restrict__ out, long ldo, int H) {
  const long t = blockIdx.x;
  float sg = 1.f;
  if (shared && shared_gate) sg = 1.f / (1.f + __expf(-shared_gate[t]));
  for (int v = threadIdx.x; v < H / 8; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int c = 0; c < k; ++c) {
      const int e = ids[t * k + c];
      if (e < e_lo || e >= e_hi) continue;
      const uint4 u = reinterpret_cast<const uint4*>(y + (t * k + c) * ldy)[v];
      const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(u2[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    if (shared) {
      const uint4 u = reinterpret_cast<const uint4*>(shared + t * lds)[v];
      const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(u2[j]);
        acc[2 * j] += f.x * sg;
        acc[2 * j + 1] += f.y * sg;
      }
    }
    if (residual) {
      const uint4 u = reinterpret_cast<const uint4*>(residual + t * ldr)[v];
      const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(u2[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    reinterpret_cast<uint4*>(out + t * ldo)[v] = o;
  }
}

int moe_combine_launch(const void* y, long ldy, const int* ids, int k, int e_lo, int e_hi, const void* shared, long lds,
                       const float* shared_gate, const void* residual, long ldr, void* out, long ldo, int T, int H,
                       cudaStream_t s) {
  if (T <= 0) return 0;
  if (H % 8) return 1;
  moe_combine_kernel<<<T, 128, 0, s>>>(static_cast<const __nv_bfloat16*>(y), ldy, ids, k, e_lo, e_hi,
                                       static_cast<const __nv_bfloat16*>(shared), lds, shared_gate,
                                       static_cast<const __nv_bfloat16*>(residual), ldr,
                                       static_cast<__nv_bfloat16*>(out), ldo, H);
  return cudaGetLastError() != cudaSuccess;
}

}  // namespace lb
