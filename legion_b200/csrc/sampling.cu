// Token selection on the device: greedy arg-max over the vocabulary (two stages, ties to the lower
// id) and temperature / min-p / top-k / top-p sampling with a counter-based RNG, so a decode step
// never ships a vocabulary-sized row to the host.
//
// Counterparts in the reference: src/cuda/sm90/cluster_select.cu (argmax_split, argmax_join) and
// the host sampler src/engine/sampling.rs (penalties -> temperature -> min-p -> top-k -> top-p).
#include "common.cuh"
#include "kernels.h"

namespace lb {

__device__ __forceinline__ void argmax_merge(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

template <typename T>
__device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__global__ void __launch_bounds__(256) argmax_part_kernel(const T* __restrict__ logits, long ld, int V, int nblk,
                                                          float* __restrict__ pv, int* __restrict__ pi) {
  const int row = blockIdx.y;
  const int per = (V + nblk - 1) / nblk;
  const int lo = blockIdx.x * per, hi = min(V, lo + per);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += 256) {
    const float v = to_f<T>(logits[row * ld + i]);
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_merge(bv, bi, ov, oi);
  }
  __shared__ float sv[8];
  __shared__ int si[8];
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) argmax_merge(bv, bi, sv[w], si[w]);
    pv[row * nblk + blockIdx.x] = bv;
    pi[row * nblk + blockIdx.x] = bi;
  }
}

__global__ void argmax_join_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int nblk,
                                   int* __restrict__ out, float* __restrict__ out_val) {
  const int row = blockIdx.x;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < nblk; i += 32) argmax_merge(bv, bi, pv[row * nblk + i], pi[row * nblk + i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_merge(bv, bi, ov, oi);
  }
  if (threadIdx.x == 0) {
    out[row] = bi;
    if (out_val) out_val[row] = bv;
  }
}

int argmax_launch(const void* logits, bool is_f32, long ld, int rows, int V, float* pv, int* pi, int nblk, int* out,
                  float* out_val, cudaStream_t s) {
  if (rows <= 0) return 0;
  dim3 grid(nblk, rows);
  if (is_f32)
    argmax_part_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(logits), ld, V, nblk, pv, pi);
  else
    argmax_part_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(logits), ld, V, nblk,
                                                           pv, pi);
  argmax_join_kernel<<<rows, 32, 0, s>>>(pv, pi, nblk, out, out_val);
  return cudaGetLastError() != cudaSuccess;
}

// ---------------------------------------------------------------------------------------------
// sampling
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

template <int THREADS>
__device__ __forceinline__ float blk_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < THREADS / 32; ++i) t += red[i];
  __syncthreads();
  return t;
}
template <int THREADS>
__device__ __forceinline__ float blk_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = -INFINITY;
  for (int i = 0; i < THREADS / 32; ++i) t = fmaxf(t, red[i]);
  __syncthreads();
  return t;
}

// One CTA per row. The kept set is {p >= thr}: thr starts at min_p * p_max, is raised by bisection
// until at most top_k entries remain, then raised again until the kept mass just covers top_p.
// The draw walks the kept entries in index order. probs_out (optional) gets the kept distribution.
__global__ void __launch_bounds__(1024) sample_kernel(const float* __restrict__ logits, long ld, int V,
                                                      const float* __restrict__ temperature,
                                                      const int* __restrict__ top_k, const float* __restrict__ top_p,
                                                      const float* __restrict__ min_p,
                                                      const unsigned long long* __restrict__ seeds,
                                                      const int* __restrict__ steps, float* __restrict__ scratch,
                                                      int* __restrict__ out) {
  constexpr int TH = 1024;
  __shared__ float red[32];
  __shared__ float s_pref[TH];
  const int row = blockIdx.x;
  const float* lg = logits + row * ld;
  float* pr = scratch + long(row) * V;
  const float temp = temperature[row];
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += TH) mx = fmaxf(mx, lg[i]);
  mx = blk_max<TH>(mx, red);
  if (temp <= 0.f) {  // greedy
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += TH)
      if (lg[i] == mx && i < bi) bi = i;
    __shared__ int s_bi;
    if (threadIdx.x == 0) s_bi = 0x7fffffff;
    __syncthreads();
    atomicMin(&s_bi, bi);
    __syncthreads();
    if (threadIdx.x == 0) out[row] = s_bi;
    return;
  }
  const float it = 1.f / temp;
  float sum = 0.f;
  for (int i = threadIdx.x; i < V; i += TH) {
    const float e = __expf((lg[i] - mx) * it);
    pr[i] = e;
    sum += e;
  }
  sum = blk_sum<TH>(sum, red);
  const float inv = 1.f / sum;
  const float pmax = inv;  // exp(0) / sum
  float thr = (min_p ? min_p[row] : 0.f) * pmax;
  const int tk = top_k ? top_k[row] : 0;
  const float tp = top_p ? top_p[row] : 1.f;
  if (tk > 0 && tk < V) {
    float lo = thr, hi = pmax;
    for (int iter = 0; iter < 30; ++iter) {
      const float mid = 0.5f * (lo + hi);
      float c = 0.f;
      for (int i = threadIdx.x; i < V; i += TH) c += (pr[i] * inv >= mid) ? 1.f : 0.f;
      c = blk_sum<TH>(c, red);
      if (c > float(tk)) lo = mid; else hi = mid;
    }
    thr = fmaxf(thr, hi);
  }
  if (tp < 1.f) {
    // largest threshold whose kept mass is still >= tp * (mass kept so far)
    float base = 0.f;
    for (int i = threadIdx.x; i < V; i += TH) { const float p = pr[i] * inv; base += (p >= thr) ? p : 0.f; }
    base = blk_sum<TH>(base, red);
    float lo = thr, hi = pmax;
    for (int iter = 0; iter < 30; ++iter) {
      const float mid = 0.5f * (lo + hi);
      float c = 0.f;
      for (int i = threadIdx.x; i < V; i += TH) { const float p = pr[i] * inv; c += (p >= mid) ? p : 0.f; }
      c = blk_sum<TH>(c, red);
      if (c >= tp * base) lo = mid; else hi = mid;
    }
    thr = fmaxf(thr, lo);
  }
  // kept mass and draw
  float kept = 0.f;
  const int per = (V + TH - 1) / TH;
  const int i0 = threadIdx.x * per, i1 = min(V, i0 + per);
  for (int i = i0; i < i1; ++i) { const float p = pr[i] * inv; kept += (p >= thr) ? p : 0.f; }
  s_pref[threadIdx.x] = kept;
  __syncthreads();
  __shared__ float s_total;
  __shared__ int s_pick;
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < TH; ++i) { const float v = s_pref[i]; s_pref[i] = t; t += v; }
    s_total = t;
    s_pick = -1;
  }
  __syncthreads();
  const uint64_t r = splitmix64(seeds[row] ^ splitmix64(uint64_t(steps ? steps[row] : 0)));
  const float u = float(r >> 40) * (1.f / 16777216.f) * s_total;
  float cum = s_pref[threadIdx.x];
  const float nxt = cum + kept;
  if (u >= cum && u < nxt) {
    int pick = -1;
    for (int i = i0; i < i1; ++i) {
      const float p = pr[i] * inv;
      if (p >= thr) {
        cum += p;
        pick = i;
        if (u < cum) break;
      }
    }
    if (pick >= 0) s_pick = pick;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (s_pick < 0) {  // numerical corner: fall back to the arg-max
      int bi = 0;
      for (int i = 0; i < V; ++i) if (lg[i] == mx) { bi = i; break; }
      s_pick = bi;
    }
    out[row] = s_pick;
  }
}

int sample_launch(const float* logits, long ld, int rows, int V, const float* temperature, const int* top_k,
                  const float* top_p, const float* min_p, const unsigned long long* seeds, const int* steps,
                  float* scratch, int* out, cudaStream_t s) {
  if (rows <= 0) return 0;
  sample_kernel<<<rows, 1024, 0, s>>>(logits, ld, V, temperature, top_k, top_p, min_p, seeds, steps, scratch, out);
  return cudaGetLastError() != cudaSuccess;
}

// logits[row, id] adjusted for presence / frequency / repetition penalties given token counts, and a
// grammar bitmask (bit = 1 keeps the token).
__global__ void penalties_mask_kernel(float* __restrict__ logits, long ld, int V, const int* __restrict__ counts,
                                      const unsigned char* __restrict__ seen, const float* __restrict__ presence,
                                      const float* __restrict__ frequency, const float* __restrict__ repetition,
                                      const unsigned int* __restrict__ mask, int mask_words) {
  const int row = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= V) return;
  float v = logits[row * ld + i];
  if (counts) {
    const int c = counts[long(row) * V + i];
    if (c > 0) v -= (presence ? presence[row] : 0.f) + (frequency ? frequency[row] : 0.f) * float(c);
  }
  if (seen && repetition && seen[long(row) * V + i]) {
    const float r = repetition[row];
    v = v > 0.f ? v / r : v * r;
  }
  if (mask && !((mask[long(row) * mask_words + (i >> 5)] >> (i & 31)) & 1u)) v = -INFINITY;
  logits[row * ld + i] = v;
}

int penalties_mask_launch(float* logits, long ld, int rows, int V, const int* counts, const unsigned char* seen,
                          const float* presence, const float* frequency, const float* repetition,
                          const unsigned int* mask, int mask_words, cudaStream_t s) {
  if (rows <= 0) return 0;
  dim3 grid((V + 255) / 256, rows);
  penalties_mask_kernel<<<grid, 256, 0, s>>>(logits, ld, V, counts, seen, presence, frequency, repetition, mask,
                                             mask_words);
  return cudaGetLastError() != cudaSuccess;
}

}  // namespace lb

// ---------------------------------------------------------------------------------------------
// Arg-max for callers that cannot allocate device memory (declared in noalloc.h).
// ---------------------------------------------------------------------------------------------
#include "noalloc.h"

namespace {

// Partial (value, index) pairs of the two-stage arg-max: LB_NOALLOC_MAX_ROWS rows x LB_NOALLOC_BLOCKS
// blocks x 8 bytes = 128 KiB, held by every device that loads this library until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[LB_NOALLOC_MAX_ROWS * LB_NOALLOC_BLOCKS * 8];

// Device address of g_noalloc_scratch per device ordinal. In host code the array's name is only a
// stand-in for the symbol, so the real address is looked up once per device with that device current.
void* g_noalloc_ptr[LB_NOALLOC_MAX_DEVICES] = {};

}  // namespace

extern "C" int lb_argmax_noalloc(const float* logits, long ld, int rows, int vocab, int* out, void* stream) {
  if (!logits || !out || rows < 0 || vocab <= 0 || ld < vocab) return LB_NOALLOC_BAD_ARGS;
  if (rows > LB_NOALLOC_MAX_ROWS) return LB_NOALLOC_TOO_LARGE;
  if (rows == 0) return LB_NOALLOC_OK;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= LB_NOALLOC_MAX_DEVICES) return LB_NOALLOC_CUDA_ERROR;
  if (!g_noalloc_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) return LB_NOALLOC_CUDA_ERROR;
    g_noalloc_ptr[dev] = p;
  }
  float* pv = static_cast<float*>(g_noalloc_ptr[dev]);
  int* pi = reinterpret_cast<int*>(pv + LB_NOALLOC_MAX_ROWS * LB_NOALLOC_BLOCKS);
  int nblk = (vocab + 4095) / 4096;
  if (nblk < 1) nblk = 1;
  if (nblk > LB_NOALLOC_BLOCKS) nblk = LB_NOALLOC_BLOCKS;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // Every partial that the join kernel reads is written by the first kernel of the same call, so
  // nothing in the scratch has to start at zero.
  lb::argmax_part_kernel<float><<<dim3(nblk, rows), 256, 0, s>>>(logits, ld, vocab, nblk, pv, pi);
  lb::argmax_join_kernel<<<rows, 32, 0, s>>>(pv, pi, nblk, out, nullptr);
  return cudaGetLastError() == cudaSuccess ? LB_NOALLOC_OK : LB_NOALLOC_CUDA_ERROR;
}
