// Gated DeltaNet: causal depthwise conv + SiLU with carried history, the gated delta rule itself
// (one CTA per (sequence, value head), state held in registers, tokens walked in order), and the
// gated RMS norm of the output. The same recurrence kernel serves decode (1 token), verify rows
// (state not written back) and commit replay (state written, outputs discarded).
//
// Per token t, value head h, key head kh:  g = exp(g_t), beta = beta_t
//   kv[c]  = sum_i S[i][c] k_i ;  delta[c] = (v_c - g * kv[c]) * beta
//   S[i][c] = g * S[i][c] + k_i * delta[c] ;  o[c] = scale * sum_i S[i][c] q_i
// with q and k L2-normalised over the head.
//
// Counterparts in the reference: src/cuda/gdn.cu (gdn_kernel, gdn_decode_kernel, gdn_keep),
// src/cuda/fused.cu (conv_silu_kernel, gated_norm_kernel), CPU form src/model/core/gdn_scan.rs.
#include "common.cuh"
#include "gdn.h"

namespace lb {

// x: [T, C] bf16; w: [C, KC] f32; conv_state: [slots, C, KC-1] f32 (oldest first). One thread per
// channel walks its sequence; the state is read at the start and (optionally) written at the end.
template <int KC>
__global__ void __launch_bounds__(128) conv1d_silu_kernel(const __nv_bfloat16* __restrict__ x, long ldx,
                                                          const float* __restrict__ w, const float* __restrict__ bias,
                                                          float* __restrict__ conv_state,
                                                          const int* __restrict__ cu_seq,
                                                          const int* __restrict__ slots, int C,
                                                          __nv_bfloat16* __restrict__ out, long ldo, int write_state) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int seq = blockIdx.y;
  if (c >= C) return;
  const int t0 = cu_seq[seq], t1 = cu_seq[seq + 1];
  const int slot = slots[seq];
  float wv[KC], h[KC - 1];
#pragma unroll
  for (int j = 0; j < KC; ++j) wv[j] = w[c * KC + j];
  float* st = conv_state + (long(slot) * C + c) * (KC - 1);
#pragma unroll
  for (int j = 0; j < KC - 1; ++j) h[j] = st[j];
  const float b = bias ? bias[c] : 0.f;
  for (int t = t0; t < t1; ++t) {
    const float xv = __bfloat162float(x[t * ldx + c]);
    float acc = b + wv[KC - 1] * xv;
#pragma unroll
    for (int j = 0; j < KC - 1; ++j) acc += wv[j] * h[j];
#pragma unroll
    for (int j = 0; j < KC - 2; ++j) h[j] = h[j + 1];
    h[KC - 2] = xv;
    out[t * ldo + c] = __float2bfloat16(acc / (1.f + __expf(-acc)));
  }
  if (write_state) {
#pragma unroll
    for (int j = 0; j < KC - 1; ++j) st[j] = h[j];
  }
}

int conv1d_silu_launch(const void* x, long ldx, const float* w, const float* bias, float* conv_state,
                       const int* cu_seq, const int* slots, int n_seqs, int C, int KC, void* out, long ldo,
                       int write_state, cudaStream_t s) {
  if (n_seqs <= 0) return 0;
  dim3 grid((C + 127) / 128, n_seqs);
#define LB_KC(K_)                                                                                              \
  if (KC == K_) {                                                                                              \
    conv1d_silu_kernel<K_><<<grid, 128, 0, s>>>(static_cast<const __nv_bfloat16*>(x), ldx, w, bias,            \
                                                conv_state, cu_seq, slots, C,                                  \
                                                static_cast<__nv_bfloat16*>(out), ldo, write_state);           \
    return cudaGetLastError() != cudaSuccess;                                                                  \
  }
  LB_KC(2) LB_KC(3) LB_KC(4) LB_KC(5) LB_KC(6) LB_KC(7) LB_KC(8)
#undef LB_KC
  return 1;
}

// qkv: [T, 2*Hk*DK + Hv*DV] bf16 as [q | k | v]; g, beta: [T, Hv] f32 (g = log decay, beta in (0,1));
// state: [slots, Hv, DK, DV] f32; out: [T, Hv, DV] bf16. 256 threads: thread (c, half) owns
// S[half*DK/2 .. , c].
template <int DK, int DV>
__global__ void __launch_bounds__(2 * DV) gdn_recurrent_kernel(
    const __nv_bfloat16* __restrict__ qkv, long ld, const float* __restrict__ g, const float* __restrict__ beta,
    float* __restrict__ state, const int* __restrict__ cu_seq, const int* __restrict__ slots, int Hk, int Hv,
    int tiled_heads, float scale, float l2_eps, __nv_bfloat16* __restrict__ out, int write_state, int write_out) {
  constexpr int HALF = DK / 2;
  const int h = blockIdx.x, seq = blockIdx.y;
  const int kh = tiled_heads ? (h % Hk) : (h / (Hv / Hk));
  const int c = threadIdx.x % DV;
  const int half = threadIdx.x / DV;
  const int t0 = cu_seq[seq], t1 = cu_seq[seq + 1];
  const int slot = slots[seq];
  __shared__ float q_s[DK], k_s[DK], part[2][DV], red[2 * DV / 32];
  __shared__ float qn_s, kn_s;
  float S[HALF];
  float* sp = state + ((long(slot) * Hv + h) * DK + half * HALF) * DV + c;
#pragma unroll
  for (int i = 0; i < HALF; ++i) S[i] = sp[long(i) * DV];
  const long q_off = long(kh) * DK, k_off = long(Hk) * DK + long(kh) * DK, v_off = 2L * Hk * DK + long(h) * DV;
  for (int t = t0; t < t1; ++t) {
    const __nv_bfloat16* row = qkv + t * ld;
    // load q, k and their squared norms
    float qq = 0.f, kk = 0.f;
    if (threadIdx.x < DK) {
      const float qv = __bfloat162float(row[q_off + threadIdx.x]);
      const float kv = __bfloat162float(row[k_off + threadIdx.x]);
      q_s[threadIdx.x] = qv;
      k_s[threadIdx.x] = kv;
      qq = qv * qv;
      kk = kv * kv;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      qq += __shfl_xor_sync(0xffffffffu, qq, o);
      kk += __shfl_xor_sync(0xffffffffu, kk, o);
    }
    if ((threadIdx.x & 31) == 0 && threadIdx.x < DK) { red[threadIdx.x >> 5] = qq; red[DK / 32 + (threadIdx.x >> 5)] = kk; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float a = 0.f, b = 0.f;
      for (int i = 0; i < DK / 32; ++i) { a += red[i]; b += red[DK / 32 + i]; }
      qn_s = rsqrtf(a + l2_eps) * scale;
      kn_s = rsqrtf(b + l2_eps);
    }
    __syncthreads();
    const float qn = qn_s, kn = kn_s;
    const float gt = __expf(g[long(t) * Hv + h]);
    const float bt = beta[long(t) * Hv + h];
    const float vc = __bfloat162float(row[v_off + c]);
    float kv = 0.f;
#pragma unroll
    for (int i = 0; i < HALF; ++i) kv += S[i] * k_s[half * HALF + i];
    part[half][c] = kv * kn;
    __syncthreads();
    const float kv_all = part[0][c] + part[1][c];
    const float delta = (vc - gt * kv_all) * bt;
    __syncthreads();
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < HALF; ++i) {
      S[i] = gt * S[i] + k_s[half * HALF + i] * kn * delta;
      o += S[i] * q_s[half * HALF + i];
    }
    part[half][c] = o * qn;
    __syncthreads();
    if (write_out && half == 0) out[(long(t) * Hv + h) * DV + c] = __float2bfloat16(part[0][c] + part[1][c]);
    __syncthreads();
  }
  if (write_state) {
#pragma unroll
    for (int i = 0; i < HALF; ++i) sp[long(i) * DV] = S[i];
  }
}

int gdn_recurrent_launch(const void* qkv, long ld, const float* g, const float* beta, float* state,
                         const int* cu_seq, const int* slots, int n_seqs, int Hk, int Hv, int DK, int DV,
                         int tiled_heads, float scale, float l2_eps, void* out, int write_state, int write_out,
                         cudaStream_t s) {
  if (n_seqs <= 0) return 0;
  dim3 grid(Hv, n_seqs);
#define LB_G(K_, V_)                                                                                               \
  if (DK == K_ && DV == V_) {                                                                                      \
    gdn_recurrent_kernel<K_, V_><<<grid, 2 * V_, 0, s>>>(static_cast<const __nv_bfloat16*>(qkv), ld, g, beta,      \
                                                         state, cu_seq, slots, Hk, Hv, tiled_heads, scale, l2_eps, \
                                                         static_cast<__nv_bfloat16*>(out), write_state, write_out);\
    return cudaGetLastError() != cudaSuccess;                                                                      \
  }
  LB_G(128, 128) LB_G(64, 64) LB_G(64, 128) LB_G(32, 32)
#undef LB_G
  return 1;
}

// g = -exp(A_log) * softplus(a + dt_bias) (A passed as -exp(A_log)), beta = sigmoid(b). a, b: [T, Hv] bf16.
__global__ void gdn_gates_kernel(const __nv_bfloat16* __restrict__ a, long lda, const __nv_bfloat16* __restrict__ b,
                                 long ldb, const float* __restrict__ A, const float* __restrict__ dt_bias, int Hv,
                                 long n, float* __restrict__ g, float* __restrict__ beta) {
  const long i = long(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long t = i / Hv;
  const int h = int(i % Hv);
  const float x = __bfloat162float(a[t * lda + h]) + dt_bias[h];
  const float sp = x > 20.f ? x : log1pf(__expf(x));
  g[i] = A[h] * sp;
  beta[i] = 1.f / (1.f + __expf(-__bfloat162float(b[t * ldb + h])));
}

int gdn_gates_launch(const void* a, long lda, const void* b, long ldb, const float* A, const float* dt_bias, int Hv,
                     long T, float* g, float* beta, cudaStream_t s) {
  const long n = T * Hv;
  if (n <= 0) return 0;
  gdn_gates_kernel<<<int((n + 255) / 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(a), lda,
                                                        static_cast<const __nv_bfloat16*>(b), ldb, A, dt_bias, Hv, n,
                                                        g, beta);
  return cudaGetLastError() != cudaSuccess;
}

// out[t, h, :] = rmsnorm(o[t, h, :]) * w * act(z[t, h, :]); act = silu (0) or sigmoid (1). Warp per (t, h).
__global__ void __launch_bounds__(128) gated_rmsnorm_kernel(const __nv_bfloat16* __restrict__ o,
                                                            const __nv_bfloat16* __restrict__ z, long ldz,
                                                            const float* __restrict__ w, float eps, int DV, int Hv,
                                                            long n_rows, int act, __nv_bfloat16* __restrict__ out) {
  const long r = (long(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (r >= n_rows) return;
  const long t = r / Hv;
  const int h = int(r % Hv);
  const __nv_bfloat16* op = o + r * DV;
  const __nv_bfloat16* zp = z + t * ldz + long(h) * DV;
  float ss = 0.f;
  for (int d = lane; d < DV; d += 32) {
    const float v = __bfloat162float(op[d]);
    ss += v * v;
  }
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, k);
  const float inv = rsqrtf(ss / float(DV) + eps);
  for (int d = lane; d < DV; d += 32) {
    const float v = __bfloat162float(op[d]) * inv * w[d];
    const float zv = __bfloat162float(zp[d]);
    const float sg = 1.f / (1.f + __expf(-zv));
    out[r * DV + d] = __float2bfloat16(v * (act == 0 ? zv * sg : sg));
  }
}

int gated_rmsnorm_launch(const void* o, const void* z, long ldz, const float* w, float eps, int DV, int Hv, long T,
                         int act, void* out, cudaStream_t s) {
  const long rows = T * Hv;
  if (rows <= 0) return 0;
  gated_rmsnorm_kernel<<<int((rows * 32 + 127) / 128), 128, 0, s>>>(static_cast<const __nv_bfloat16*>(o),
                                                                    static_cast<const __nv_bfloat16*>(z), ldz, w, eps,
                                                                    DV, Hv, rows, act,
                                                                    static_cast<__nv_bfloat16*>(out));
  return cudaGetLastError() != cudaSuccess;
}

}  // namespace lb
