// Mamba-2 (SSD) state-space recurrence for decode steps and prompt chunks, one CTA per (head, sequence):
//
//   dt  = softplus(dt_raw[t, h] + dt_bias[h]),  dA = exp(dt * A[h])
//   S[d, s]  = S[d, s] * dA + dt * x[t, h, d] * B[t, g, s]
//   y[t, h, d] = (sum_s S[d, s] * C[t, g, s] + D[h] * x[t, h, d]) * silu(z[t, h, d])
//
// The fp32 state of a (sequence, head) stays in registers for the whole chunk (thread (d, j) owns ds / W consecutive
// state columns of row d, W = 256 / head_dim threads per row, the y reduction is W lanes wide), B and C rows of a
// token are staged in shared memory for all rows, and the gate by silu(z) rides on the write. The RMSNorm over the
// whole inner width follows as the ordinary norm kernel.
//
// Counterpart in the reference: the Mamba-2 scan of src/model/nemotron_h.rs / src/cuda (selective scan, decode and
// chunk forms).
#include "common.cuh"
#include "kernels.h"

namespace lb {
namespace {

constexpr int MAXPT = 32;      // state columns per thread

__global__ void __launch_bounds__(256) mamba2_scan_kernel(
    const __nv_bfloat16* __restrict__ xbc, long ldx,       // [T, di + 2 * ng * ds]: x | B | C (after the causal conv)
    const __nv_bfloat16* __restrict__ dt_raw, long lddt,   // [T, nh]
    const __nv_bfloat16* __restrict__ z, long ldz,         // [T, di]
    const float* __restrict__ A, const float* __restrict__ Dp, const float* __restrict__ dt_bias,
    float* __restrict__ state,                             // [slots, nh, hd, ds]
    const int* __restrict__ cu_seq, const int* __restrict__ slots, int nh, int hd, int ng, int ds,
    __nv_bfloat16* __restrict__ y, long ldy, int write_state) {
  extern __shared__ float sh[];                             // B row | C row of the current token
  griddep_wait();
  griddep_launch();
  const int h = blockIdx.x, seq = blockIdx.y;
  const int W = 256 / hd;                                   // threads per state row
  const int cnt = ds / W;                                   // state columns per thread
  const int d = threadIdx.x / W, j = threadIdx.x % W;
  const int g = h / (nh / ng);
  const int di = nh * hd;
  const int t0 = cu_seq[seq], t1 = cu_seq[seq + 1];
  const int slot = slots[seq];
  if (t1 <= t0 || slot < 0) return;
  float* S = state + ((long(slot) * nh + h) * hd + d) * ds + j * cnt;
  float s[MAXPT];
#pragma unroll
  for (int i = 0; i < MAXPT; ++i) s[i] = i < cnt ? S[i] : 0.f;
  const float a = A[h], dd = Dp[h], db = dt_bias[h];
  float* sB = sh;
  float* sC = sh + ds;
  for (int t = t0; t < t1; ++t) {
    const __nv_bfloat16* row = xbc + long(t) * ldx;
    __syncthreads();                                        // the previous token's B / C are no longer read
    for (int i = threadIdx.x; i < 2 * ds; i += 256)
      sh[i] = __bfloat162float(row[di + (i < ds ? g * ds + i : ng * ds + g * ds + (i - ds))]);
    __syncthreads();
    const float raw = __bfloat162float(dt_raw[long(t) * lddt + h]) + db;
    const float dt = raw > 20.f ? raw : log1pf(__expf(raw));
    const float dA = __expf(dt * a);
    const float xv = __bfloat162float(row[h * hd + d]);
    const float dx = dt * xv;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < MAXPT; ++i) {
      if (i < cnt) {
        s[i] = fmaf(s[i], dA, dx * sB[j * cnt + i]);
        acc = fmaf(s[i], sC[j * cnt + i], acc);
      }
    }
    for (int o = W >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (j == 0) {
      const float zv = __bfloat162float(z[long(t) * ldz + h * hd + d]);
      const float out = (acc + dd * xv) * (zv / (1.f + __expf(-zv)));
      y[long(t) * ldy + h * hd + d] = __float2bfloat16(out);
    }
  }
  if (write_state) {
#pragma unroll
    for (int i = 0; i < MAXPT; ++i)
      if (i < cnt) S[i] = s[i];
  }
}

}  // namespace

int mamba2_scan_launch(const void* xbc, long ldx, const void* dt_raw, long lddt, const void* z, long ldz, const float* A,
                       const float* D, const float* dt_bias, float* state, const int* cu_seq, const int* slots,
                       int n_seqs, int nh, int hd, int ng, int ds, void* y, long ldy, int write_state, cudaStream_t s) {
  if (n_seqs <= 0) return 0;
  // thread (d, j): 256 / hd threads per state row, each with ds / W columns in registers, W lanes inside one warp
  if (hd <= 0 || hd > 256 || (256 % hd) || (hd & (hd - 1))) return 1;
  const int W = 256 / hd;
  if (W > 32 || ds % W || ds / W > MAXPT || nh % ng) return 1;
  launch_pdl(mamba2_scan_kernel, dim3(nh, n_seqs), dim3(256), size_t(2 * ds) * sizeof(float), s,
             static_cast<const __nv_bfloat16*>(xbc), ldx, static_cast<const __nv_bfloat16*>(dt_raw), lddt,
             static_cast<const __nv_bfloat16*>(z), ldz, A, D, dt_bias, state, cu_seq, slots, nh, hd, ng, ds,
             static_cast<__nv_bfloat16*>(y), ldy, write_state);
  return cudaGetLastError() != cudaSuccess;
}

}  // namespace lb
