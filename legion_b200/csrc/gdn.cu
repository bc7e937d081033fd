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

// Prompt-sized form: tokens in parallel. A CTA covers 128 channels x TOK consecutive tokens of one sequence; a thread
// walks its channel over those tokens with the KC - 1 previous inputs in registers (taken from the tensor itself, or
// from the carried history for the first tokens of the sequence). The CTA that holds the sequence's last token
// writes the new history. Reads of x are coalesced across the 128 channels of a token row.
template <int KC>
__global__ void __launch_bounds__(128) conv1d_silu_prompt_kernel(const __nv_bfloat16* __restrict__ x, long ldx,
                                                                 const float* __restrict__ w,
                                                                 const float* __restrict__ bias,
                                                                 float* __restrict__ conv_state,
                                                                 const int* __restrict__ cu_seq,
                                                                 const int* __restrict__ slots, int C, int tok_per_cta,
                                                                 __nv_bfloat16* __restrict__ out, long ldo,
                                                                 int write_state) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int seq = blockIdx.z;
  const int t0 = cu_seq[seq], t1 = cu_seq[seq + 1];
  const int ta = t0 + blockIdx.y * tok_per_cta;
  if (c >= C || ta >= t1) return;
  const int tb = min(t1, ta + tok_per_cta);
  const int slot = slots[seq];
  float wv[KC], h[KC - 1];
#pragma unroll
  for (int j = 0; j < KC; ++j) wv[j] = w[c * KC + j];
  float* st = conv_state + (long(slot) * C + c) * (KC - 1);
  // h[j] = input of token ta - (KC - 1) + j: from x when that token belongs to this step, else from the history
#pragma unroll
  for (int j = 0; j < KC - 1; ++j) {
    const int t = ta - (KC - 1) + j;
    h[j] = t >= t0 ? __bfloat162float(x[long(t) * ldx + c]) : st[(KC - 1) + (t - t0)];
  }
  const float b = bias ? bias[c] : 0.f;
  for (int t = ta; t < tb; ++t) {
    const float xv = __bfloat162float(x[long(t) * ldx + c]);
    float acc = b + wv[KC - 1] * xv;
#pragma unroll
    for (int j = 0; j < KC - 1; ++j) acc += wv[j] * h[j];
#pragma unroll
    for (int j = 0; j < KC - 2; ++j) h[j] = h[j + 1];
    h[KC - 2] = xv;
    out[long(t) * ldo + c] = __float2bfloat16(acc / (1.f + __expf(-acc)));
  }
  (void)write_state;   // the history is replaced by conv1d_state_kernel after this kernel
}

// History update of the prompt form: one thread per (sequence, channel) after the main kernel.
template <int KC>
__global__ void __launch_bounds__(128) conv1d_state_kernel(const __nv_bfloat16* __restrict__ x, long ldx,
                                                           float* __restrict__ conv_state,
                                                           const int* __restrict__ cu_seq,
                                                           const int* __restrict__ slots, int C) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int seq = blockIdx.y;
  if (c >= C) return;
  const int t0 = cu_seq[seq], t1 = cu_seq[seq + 1];
  if (t1 <= t0) return;
  float* st = conv_state + (long(slots[seq]) * C + c) * (KC - 1);
  float h[KC - 1];
#pragma unroll
  for (int j = 0; j < KC - 1; ++j) {
    const int t = t1 - (KC - 1) + j;
    h[j] = t >= t0 ? __bfloat162float(x[long(t) * ldx + c]) : st[(KC - 1) + (t - t0)];
  }
#pragma unroll
  for (int j = 0; j < KC - 1; ++j) st[j] = h[j];
}

int conv1d_silu_launch(const void* x, long ldx, const float* w, const float* bias, float* conv_state,
                       const int* cu_seq, const int* slots, int n_seqs, int C, int KC, void* out, long ldo,
                       int write_state, cudaStream_t s, int max_len) {
  if (n_seqs <= 0) return 0;
  auto xb = static_cast<const __nv_bfloat16*>(x);
  auto ob = static_cast<__nv_bfloat16*>(out);
  if (max_len >= 64) {
    // prompt rows: tokens in parallel, then the history update as a second small launch (stream order keeps the
    // main kernel's reads of the old history before its replacement)
    const int tok = 32;
    dim3 grid((C + 127) / 128, (max_len + tok - 1) / tok, n_seqs), grid2((C + 127) / 128, n_seqs);
#define LB_KCP(K_)                                                                                             \
  if (KC == K_) {                                                                                              \
    conv1d_silu_prompt_kernel<K_><<<grid, 128, 0, s>>>(xb, ldx, w, bias, conv_state, cu_seq, slots, C, tok, ob, \
                                                       ldo, write_state);                                      \
    if (write_state) conv1d_state_kernel<K_><<<grid2, 128, 0, s>>>(xb, ldx, conv_state, cu_seq, slots, C);      \
    return cudaGetLastError() != cudaSuccess;                                                                  \
  }
    LB_KCP(2) LB_KCP(3) LB_KCP(4) LB_KCP(5) LB_KCP(6) LB_KCP(7) LB_KCP(8)
#undef LB_KCP
    return 1;
  }
  dim3 grid((C + 127) / 128, n_seqs);
#define LB_KC(K_)                                                                                              \
  if (KC == K_) {                                                                                              \
    conv1d_silu_kernel<K_><<<grid, 128, 0, s>>>(xb, ldx, w, bias, conv_state, cu_seq, slots, C, ob, ldo,       \
                                                write_state);                                                  \
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

// Prompt-sized recurrence: one state COLUMN per thread. The columns of S (fixed value index c) evolve independently
// given k, q, beta, g, so a thread that keeps S[:, c] in registers (DK floats) needs no cross-thread reduction at
// all: kv = S[:, c] . k, delta, rank-1 update and o = S[:, c] . q are thread-local. A CTA is two warps: warp 0 owns
// 32 columns of one value head, warp 1 stages chunks of 8 tokens ahead (loads q, k, v, g, beta, L2-normalises q and
// k, converts to fp32) into a double-buffered shared-memory ring, so the consumer never waits for global memory.
// Grid = (value heads x DV / 32, sequences): 4x the CTAs of the decode kernel and no block-wide barriers per token.
template <int DK>
__global__ void __launch_bounds__(64) gdn_scan_cols_kernel(
    const __nv_bfloat16* __restrict__ qkv, long ld, const float* __restrict__ g, const float* __restrict__ beta,
    float* __restrict__ state, const int* __restrict__ cu_seq, const int* __restrict__ slots, int Hk, int Hv, int DV,
    int tiled_heads, float scale, float l2_eps, __nv_bfloat16* __restrict__ out, int write_state, int write_out) {
  constexpr int CH = 8;
  constexpr int PER = DK / 32;                  // q / k elements per producer lane
  __shared__ __align__(16) float q_s[2][CH][DK];
  __shared__ __align__(16) float k_s[2][CH][DK];
  __shared__ float v_s[2][CH][32];
  __shared__ float g_s[2][CH], b_s[2][CH];
  const int tiles = DV / 32;
  const int h = blockIdx.x / tiles, c0 = (blockIdx.x % tiles) * 32;
  const int seq = blockIdx.y;
  const int kh = tiled_heads ? (h % Hk) : (h / (Hv / Hk));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = cu_seq[seq], t1 = cu_seq[seq + 1];
  const int n_chunks = (t1 - t0 + CH - 1) / CH;
  const long q_off = long(kh) * DK, k_off = long(Hk) * DK + long(kh) * DK, v_off = 2L * Hk * DK + long(h) * DV + c0;
  // named barriers: 1 + buf = "chunk buf filled", 3 + buf = "chunk buf consumed"
  if (warp == 1) {
    for (int ck = 0; ck < n_chunks; ++ck) {
      const int buf = ck & 1;
      if (ck >= 2) asm volatile("bar.sync %0, 64;" ::"r"(3 + buf) : "memory");
      float qv[CH][PER], kv[CH][PER], vv[CH];
#pragma unroll
      for (int j = 0; j < CH; ++j) {            // all loads of the chunk are in flight together
        const int t = t0 + ck * CH + j;
        const bool ok = t < t1;
        const __nv_bfloat16* row = qkv + long(ok ? t : t0) * ld;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
          qv[j][i] = ok ? __bfloat162float(row[q_off + lane + 32 * i]) : 0.f;
          kv[j][i] = ok ? __bfloat162float(row[k_off + lane + 32 * i]) : 0.f;
        }
        vv[j] = ok ? __bfloat162float(row[v_off + lane]) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int t = t0 + ck * CH + j;
        float qq = 0.f, kk = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) { qq += qv[j][i] * qv[j][i]; kk += kv[j][i] * kv[j][i]; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          qq += __shfl_xor_sync(0xffffffffu, qq, o);
          kk += __shfl_xor_sync(0xffffffffu, kk, o);
        }
        const float qn = rsqrtf(qq + l2_eps) * scale, kn = rsqrtf(kk + l2_eps);
#pragma unroll
        for (int i = 0; i < PER; ++i) {
          q_s[buf][j][lane + 32 * i] = qv[j][i] * qn;
          k_s[buf][j][lane + 32 * i] = kv[j][i] * kn;
        }
        v_s[buf][j][lane] = vv[j];
        if (lane == 0) {
          g_s[buf][j] = t < t1 ? __expf(g[long(t) * Hv + h]) : 1.f;
          b_s[buf][j] = t < t1 ? beta[long(t) * Hv + h] : 0.f;
        }
      }
      __threadfence_block();
      asm volatile("bar.arrive %0, 64;" ::"r"(1 + buf) : "memory");
    }
  } else {
    float S[DK];
    const int slot = slots[seq];
    float* sp = state + ((long(slot) * Hv + h) * DK) * DV + c0 + lane;
#pragma unroll
    for (int i = 0; i < DK; ++i) S[i] = sp[long(i) * DV];
    for (int ck = 0; ck < n_chunks; ++ck) {
      const int buf = ck & 1;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + buf) : "memory");
      const int nt = min(CH, t1 - t0 - ck * CH);
      for (int j = 0; j < nt; ++j) {
        const float gt = g_s[buf][j], bt = b_s[buf][j], vc = v_s[buf][j][lane];
        const float4* k4 = reinterpret_cast<const float4*>(k_s[buf][j]);
        const float4* q4 = reinterpret_cast<const float4*>(q_s[buf][j]);
        // four independent accumulators per dot product: the FMA chains are the critical path of a single warp
        float kv0 = 0.f, kv1 = 0.f, kv2 = 0.f, kv3 = 0.f;
#pragma unroll
        for (int i = 0; i < DK / 4; ++i) {
          const float4 kq = k4[i];
          kv0 = fmaf(S[4 * i], kq.x, kv0);
          kv1 = fmaf(S[4 * i + 1], kq.y, kv1);
          kv2 = fmaf(S[4 * i + 2], kq.z, kv2);
          kv3 = fmaf(S[4 * i + 3], kq.w, kv3);
        }
        const float kvd = (kv0 + kv1) + (kv2 + kv3);
        const float delta = (vc - gt * kvd) * bt;
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
        for (int i = 0; i < DK / 4; ++i) {
          const float4 kq = k4[i];
          const float4 qq = q4[i];
          S[4 * i] = fmaf(gt, S[4 * i], kq.x * delta);
          S[4 * i + 1] = fmaf(gt, S[4 * i + 1], kq.y * delta);
          S[4 * i + 2] = fmaf(gt, S[4 * i + 2], kq.z * delta);
          S[4 * i + 3] = fmaf(gt, S[4 * i + 3], kq.w * delta);
          o0 = fmaf(S[4 * i], qq.x, o0);
          o1 = fmaf(S[4 * i + 1], qq.y, o1);
          o2 = fmaf(S[4 * i + 2], qq.z, o2);
          o3 = fmaf(S[4 * i + 3], qq.w, o3);
        }
        const float o = (o0 + o1) + (o2 + o3);
        if (write_out) out[(long(t0 + ck * CH + j) * Hv + h) * DV + c0 + lane] = __float2bfloat16(o);
      }
      if (ck + 2 < n_chunks) asm volatile("bar.arrive %0, 64;" ::"r"(3 + buf) : "memory");
    }
    if (write_state) {
#pragma unroll
      for (int i = 0; i < DK; ++i) sp[long(i) * DV] = S[i];
    }
  }
}

int gdn_recurrent_launch(const void* qkv, long ld, const float* g, const float* beta, float* state,
                         const int* cu_seq, const int* slots, int n_seqs, int Hk, int Hv, int DK, int DV,
                         int tiled_heads, float scale, float l2_eps, void* out, int write_state, int write_out,
                         int prompt_rows, cudaStream_t s) {
  if (n_seqs <= 0) return 0;
  if (prompt_rows && (DK == 128 || DK == 64) && DV % 32 == 0) {
    dim3 grid2(Hv * (DV / 32), n_seqs);
    if (DK == 128)
      gdn_scan_cols_kernel<128><<<grid2, 64, 0, s>>>(static_cast<const __nv_bfloat16*>(qkv), ld, g, beta, state, cu_seq,
                                                     slots, Hk, Hv, DV, tiled_heads, scale, l2_eps,
                                                     static_cast<__nv_bfloat16*>(out), write_state, write_out);
    else
      gdn_scan_cols_kernel<64><<<grid2, 64, 0, s>>>(static_cast<const __nv_bfloat16*>(qkv), ld, g, beta, state, cu_seq,
                                                    slots, Hk, Hv, DV, tiled_heads, scale, l2_eps,
                                                    static_cast<__nv_bfloat16*>(out), write_state, write_out);
    return cudaGetLastError() != cudaSuccess;
  }
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

// Decode step of a Gated DeltaNet layer in ONE launch: causal conv + SiLU of this token's q / k / v channels (with
// the carried history), gates, the delta-rule update of the state, and the gated RMS norm of the output. One CTA
// per (key head, sequence) serves the r = Hv / Hk value heads that share the key head (256 threads each), so the
// q / k convolution, their L2 norms and the conv-history update are done once and nobody reads a history another
// CTA is rewriting. Every sequence contributes exactly one token (row `seq` of proj).
//   proj row = [q (Hk*DK) | k (Hk*DK) | v (Hv*DV) | z (Hv*DV) | b (Hv) | a (Hv)]  (the fused input projection)
// Intermediate values are rounded to bf16 where the separate kernels store them as bf16 (conv outputs, the
// recurrence output), so a decode step gives the same numbers as the multi-kernel path used for verify rows.
template <int DK, int DV, int KC>
__global__ void __launch_bounds__(1024) gdn_decode_fused_kernel(
    const __nv_bfloat16* __restrict__ proj, long ld, const float* __restrict__ conv_w, float* __restrict__ conv_state,
    const float* __restrict__ A, const float* __restrict__ dt_bias, const float* __restrict__ norm_w, float eps,
    int act, float* __restrict__ state, const int* __restrict__ slots, int Hk, int Hv, int tiled_heads, float scale,
    float l2_eps, __nv_bfloat16* __restrict__ out) {
  static_assert(DK == DV, "thread layout assumes square heads");
  constexpr int HALF = DK / 2;
  constexpr int GT = 2 * DV;                     // threads per value head
  constexpr int MAXR = 4;
  griddep_wait();
  griddep_launch();
  const int kh = blockIdx.x, seq = blockIdx.y;
  const int r = Hv / Hk;
  const int j = threadIdx.x / GT, tid = threadIdx.x % GT;
  const int h = tiled_heads ? kh + j * Hk : kh * r + j;
  const int c = tid % DV, half = tid / DV;
  const int C = 2 * Hk * DK + Hv * DV;
  const int slot = slots[seq];
  const __nv_bfloat16* row = proj + long(seq) * ld;
  __shared__ float q_s[DK], k_s[DK], v_s[MAXR][DV], part[MAXR][2][DV], red[2 * DK / 32], red2[MAXR][DV / 32];
  __shared__ float qn_s, kn_s;
  // state of this thread's half column: the loads are in flight while the convolution runs
  float S[HALF];
  float* sp = state + ((long(slot) * Hv + h) * DK + half * HALF) * DV + c;
#pragma unroll
  for (int i = 0; i < HALF; ++i) S[i] = sp[long(i) * DV];

  auto conv = [&](int ch) -> float {
    float wv[KC], hh[KC - 1];
#pragma unroll
    for (int i = 0; i < KC; ++i) wv[i] = conv_w[ch * KC + i];
    float* st = conv_state + (long(slot) * C + ch) * (KC - 1);
#pragma unroll
    for (int i = 0; i < KC - 1; ++i) hh[i] = st[i];
    const float xv = __bfloat162float(row[ch]);
    float acc = wv[KC - 1] * xv;
#pragma unroll
    for (int i = 0; i < KC - 1; ++i) acc += wv[i] * hh[i];
#pragma unroll
    for (int i = 0; i < KC - 2; ++i) st[i] = hh[i + 1];
    st[KC - 2] = xv;
    return __bfloat162float(__float2bfloat16(acc / (1.f + __expf(-acc))));
  };
  float qq = 0.f, kk = 0.f;
  if (j == 0) {
    // threads 0 .. DK-1: q channel, DK .. 2 DK-1: k channel of this key head
    const float v = conv((half == 0 ? 0 : Hk * DK) + kh * DK + c);
    if (half == 0) { q_s[c] = v; qq = v * v; } else { k_s[c] = v; kk = v * v; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      qq += __shfl_xor_sync(0xffffffffu, qq, o);
      kk += __shfl_xor_sync(0xffffffffu, kk, o);
    }
    if ((tid & 31) == 0) red[tid >> 5] = half == 0 ? qq : kk;
  }
  if (half == 0) v_s[j][c] = conv(2 * Hk * DK + h * DV + c);
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f, b = 0.f;
    for (int i = 0; i < DK / 32; ++i) { a += red[i]; b += red[DK / 32 + i]; }
    qn_s = rsqrtf(a + l2_eps) * scale;
    kn_s = rsqrtf(b + l2_eps);
  }
  // gates of this value head (every thread computes them: two loads and a few operations)
  const float av = __bfloat162float(row[C + Hv * DV + Hv + h]) + dt_bias[h];
  const float spv = av > 20.f ? av : log1pf(__expf(av));
  const float gt = __expf(A[h] * spv);
  const float bt = 1.f / (1.f + __expf(-__bfloat162float(row[C + Hv * DV + h])));
  __syncthreads();
  const float qn = qn_s, kn = kn_s;
  float kv = 0.f;
#pragma unroll
  for (int i = 0; i < HALF; ++i) kv += S[i] * k_s[half * HALF + i];
  part[j][half][c] = kv * kn;
  __syncthreads();
  const float delta = (v_s[j][c] - gt * (part[j][0][c] + part[j][1][c])) * bt;
  __syncthreads();
  float o = 0.f;
#pragma unroll
  for (int i = 0; i < HALF; ++i) {
    S[i] = gt * S[i] + k_s[half * HALF + i] * kn * delta;
    o += S[i] * q_s[half * HALF + i];
  }
  part[j][half][c] = o * qn;
#pragma unroll
  for (int i = 0; i < HALF; ++i) sp[long(i) * DV] = S[i];
  __syncthreads();
  // gated RMS norm over the head's DV outputs
  float ov = 0.f, ss = 0.f;
  if (half == 0) {
    ov = __bfloat162float(__float2bfloat16(part[j][0][c] + part[j][1][c]));
    ss = ov * ov;
#pragma unroll
    for (int k = 16; k > 0; k >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, k);
    if ((c & 31) == 0) red2[j][c >> 5] = ss;
  }
  __syncthreads();
  if (half == 0) {
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < DV / 32; ++i) tot += red2[j][i];
    const float inv = rsqrtf(tot / float(DV) + eps);
    const float zv = __bfloat162float(row[C + h * DV + c]);
    const float sg = 1.f / (1.f + __expf(-zv));
    out[(long(seq) * Hv + h) * DV + c] = __float2bfloat16(ov * inv * norm_w[c] * (act == 0 ? zv * sg : sg));
  }
}

int gdn_decode_fused_launch(const void* proj, long ld, const float* conv_w, float* conv_state, int KC, const float* A,
                            const float* dt_bias, const float* norm_w, float eps, int act, float* state,
                            const int* slots, int n_seqs, int Hk, int Hv, int DK, int DV, int tiled_heads, float scale,
                            float l2_eps, void* out, cudaStream_t s) {
  if (n_seqs <= 0) return 0;
  if (Hk <= 0 || Hv % Hk || Hv / Hk > 4 || KC != 4) return 1;
  const int r = Hv / Hk;
  dim3 grid(Hk, n_seqs);
#define LB_GF(D_)                                                                                                   \
  if (DK == D_ && DV == D_) {                                                                                       \
    launch_pdl(gdn_decode_fused_kernel<D_, D_, 4>, grid, dim3(2 * D_ * r), 0, s,                                    \
               static_cast<const __nv_bfloat16*>(proj), ld, conv_w, conv_state, A, dt_bias, norm_w, eps, act, state, \
               slots, Hk, Hv, tiled_heads, scale, l2_eps, static_cast<__nv_bfloat16*>(out));                        \
    return cudaGetLastError() != cudaSuccess;                                                                       \
  }
  LB_GF(128) LB_GF(64)
#undef LB_GF
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
