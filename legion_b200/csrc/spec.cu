// Small device kernels of the sampling / speculative-decoding tail of a step, so that a decode or verify step
// can stay on the device (inside the step's CUDA graph) until one packed result is copied to the host.
//   token_logprobs   log-probability of the chosen token of every row + the top-n alternatives
//   spec_accept      greedy acceptance of draft tokens against the target's arg-max rows (prefix + bonus token)
//   gather_rows_i32  verify-row index list from (cu_q, keep) for logits selection
// Counterparts in the reference: host sampling.rs / accept logic in src/spec/mod.rs, src/cuda/mtp_cond.cu (device
// "continue drafting" flag), src/cuda/cluster_select.cu.
#include "common.cuh"
#include "kernels.h"

namespace lb {

// One CTA (256 threads) per row. lse by two block reductions; top-n by n rounds of block arg-max over the row
// (n <= 20, rows are L2 resident after the first pass); ties go to the lower token id.
__global__ void __launch_bounds__(256) token_logprobs_kernel(const float* __restrict__ logits, long ld, int V,
                                                             const int* __restrict__ chosen, int n_top,
                                                             float* __restrict__ chosen_lp,
                                                             int* __restrict__ top_ids, float* __restrict__ top_lp) {
  __shared__ float red[8];
  __shared__ int redi[8];
  __shared__ int picked[20];
  __shared__ float s_lse;
  griddep_wait();
  const int row = blockIdx.x;
  const float* lg = logits + long(row) * ld;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += 256) mx = fmaxf(mx, lg[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) mx = fmaxf(mx, red[i]);
  __syncthreads();
  float sum = 0.f;
  for (int i = threadIdx.x; i < V; i += 256) sum += __expf(lg[i] - mx);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += red[i];
    s_lse = mx + __logf(t);
    chosen_lp[row] = lg[chosen[row]] - s_lse;
  }
  __syncthreads();
  const float lse = s_lse;
  for (int r = 0; r < n_top; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += 256) {
      const float v = lg[i];
      if (v > bv || (v == bv && i < bi)) {
        bool taken = false;
        for (int j = 0; j < r; ++j) taken |= (picked[j] == i);
        if (!taken) { bv = v; bi = i; }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { red[warp] = bv; redi[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int i = 1; i < 8; ++i)
        if (red[i] > bv || (red[i] == bv && redi[i] < bi)) { bv = red[i]; bi = redi[i]; }
      picked[r] = bi;
      top_ids[row * n_top + r] = bi;
      top_lp[row * n_top + r] = bv - lse;
    }
    __syncthreads();
  }
}

int token_logprobs_launch(const float* logits, long ld, int rows, int V, const int* chosen, int n_top,
                          float* chosen_lp, int* top_ids, float* top_lp, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (n_top < 0 || n_top > 20) return 1;
  return launch_pdl(token_logprobs_kernel, dim3(rows), dim3(256), 0, s, logits, ld, V, chosen, n_top, chosen_lp,
                    top_ids, top_lp) != cudaSuccess;
}

// Greedy verification. Sequence b fed (1 + n_draft[b]) rows starting at row cu[b]: row j holds the target's arg-max
// after the tokens up to draft j. Draft j (0-based) is accepted while target[cu[b] + j] == draft[b][j]; the token
// emitted after the accepted prefix is target[cu[b] + accepted] (the "bonus"). One thread per sequence (k is tiny).
__global__ void spec_accept_kernel(const int* __restrict__ target, const int* __restrict__ cu,
                                   const int* __restrict__ draft, int max_draft, const int* __restrict__ n_draft,
                                   int B, int* __restrict__ accepted, int* __restrict__ bonus,
                                   int* __restrict__ any_rejected) {
  griddep_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const int base = cu[b], nd = n_draft[b];
  int a = 0;
  while (a < nd && target[base + a] == draft[b * max_draft + a]) ++a;
  accepted[b] = a;
  bonus[b] = target[base + a];
  if (a < nd && any_rejected) atomicOr(any_rejected, 1);
}

int spec_accept_launch(const int* target, const int* cu, const int* draft, int max_draft, const int* n_draft, int B,
                       int* accepted, int* bonus, int* any_rejected, cudaStream_t s) {
  if (B <= 0) return 0;
  return launch_pdl(spec_accept_kernel, dim3((B + 127) / 128), dim3(128), 0, s, target, cu, draft, max_draft, n_draft,
                    B, accepted, bonus, any_rejected) != cudaSuccess;
}

}  // namespace lb
