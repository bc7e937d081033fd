// Chunked Gated DeltaNet scan for prompt-sized steps on tcgen05 tensor cores (64-token chunks, WY / UT form).
//
// Per value head, with decay a_t = exp(g_t), the recurrence  S_t = a_t S_{t-1} + k_t d_t^T,
// d_t = b_t (v_t - a_t S_{t-1}^T k_t),  o_t = S_t^T q_t  is rewritten per chunk of C = 64 tokens with the cumulative
// decay c_i = sum_{j<=i} g_j (inside the chunk):
//     A_ij  = b_i exp(c_i - c_j) (k_i . k_j)            (j < i, strictly lower triangular)
//     T     = (I + A)^-1                                 (unit lower triangular)
//     U     = T diag(b) V            W = T diag(b exp(c)) K
//     M_ij  = exp(c_i - c_j) (q_i . k_j)                 (j <= i)
//     D     = U - W S_0              O = diag(exp(c)) Q S_0 + M D
//     S_C   = exp(c_C) S_0 + (diag(exp(c_C - c)) K)^T D
// Everything that does not involve the state (A, T, U, W, M, the scaled copies of K and Q) is computed for all
// chunks in parallel by the PREP kernel: one CTA per (128-token block = two chunks, value head); K K^T, Q K^T, T V and
// T K are 128 x 128 x 128 tcgen05 MMAs over TMA-loaded tiles (the block-diagonal T covers both chunks), the 64 x 64
// triangular inverses run on CUDA cores between them (thread = column, forward substitution over broadcast
// shared-memory reads).  The SCAN kernel then walks the chunks of a sequence in order, one CTA per (value head,
// sequence), in the transposed form that makes every operand natural for UMMA: the state S^T [dv, dk] and the
// correction D^T [dv, tokens] are A operands that the worker threads (thread = dv row = TMEM lane) write as K-major
// 128-byte-swizzled rows, the per-chunk tiles W, Q', M arrive by TMA as K-major B operands and K' as an MN-major B
// operand.  The fp32 state lives in tensor memory for the whole sequence (pre-multiplied by the next chunk's decay so
// that the update MMA accumulates onto it) and is rounded to bf16 only as an MMA operand.
//
// q and k are L2-normalised per row (q also carries the softmax-free scale); the norms are folded into the
// elementwise factors above, so the tiles are used as loaded.
//
// Counterpart in the reference: src/cuda/gdn_mma.cu (gdn_single / gdn_staged / gdn_split: 16-token chunks on
// mma.sync), oracle src/model/core/gdn_scan.rs.
#include "common.cuh"
#include "gdn.h"
#include "tmap.cuh"

namespace lb {
namespace {

constexpr int CH = 64;          // chunk
constexpr int BLK = 128;        // tokens per prep CTA (two chunks)
constexpr int D = 128;          // head dim (dk = dv)
constexpr int HALF_BYTES = BLK * 128;     // one 64-column half of a 128-row bf16 tile

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),
      "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// element (row, col) of a K-major 128-byte-swizzled bf16 tile made of 64-column halves of `rows` rows each
__device__ __forceinline__ uint32_t sw_off(int rows, int row, int col) {
  return uint32_t((col >> 6) * (rows * 128) + row * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4) + ((col & 7) << 1));
}

struct PrepArgs {
  const float* g; const float* beta;      // [T, Hv]
  const int* blk_t0; const int* blk_n;    // per 128-token block: first token row, valid tokens (1..128)
  int Hk, Hv, tiled_heads;
  float scale, l2_eps;
  __nv_bfloat16* U; __nv_bfloat16* W; __nv_bfloat16* Kd; __nv_bfloat16* Qg;   // [items * 128, 128]
  __nv_bfloat16* M;                       // [items * 128, 64]
  float* gC;                              // [items * 2] decay of each chunk
  int* status;
};

// ---------------------------------------------------------------------------------------------------------------
// PREP: grid (blocks, value heads), 160 threads: warps 0..3 = workers (thread = token row), warp 4 = TMA + MMA.
// ---------------------------------------------------------------------------------------------------------------
constexpr int PREP_A_STRIDE = 68;   // floats per row of the fp32 A scratch
constexpr int PREP_SMEM = 4 * 2 * HALF_BYTES + 2 * CH * PREP_A_STRIDE * 4 + 4 * 128 * 4 + 1024 + 256;

__global__ void __launch_bounds__(160, 1)
gdn_chunk_prep_kernel(const __grid_constant__ CUtensorMap tmQKV, const PrepArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;                                  // [2][128][128 B]
  uint8_t* k_s = q_s + 2 * HALF_BYTES;
  uint8_t* v_s = k_s + 2 * HALF_BYTES;
  uint8_t* t_s = v_s + 2 * HALF_BYTES;                  // T' as A operand: [2 token halves][128 rows][128 B]
  float* a_s = reinterpret_cast<float*>(t_s + 2 * HALF_BYTES);          // [2][64][68]
  float* cs_s = a_s + 2 * CH * PREP_A_STRIDE;           // [128] cumulative log decay inside the chunk
  float* be_s = cs_s + 128;                             // [128] beta (0 for padding rows)
  float* qn_s = be_s + 128;                             // [128] 1 / |q| * scale
  float* kn_s = qn_s + 128;                             // [128] 1 / |k|
  uint64_t* bars = reinterpret_cast<uint64_t*>(kn_s + 128);
  uint64_t* ld_full = bars;        // TMA landed
  uint64_t* s_done = bars + 1;     // K K^T, Q K^T done
  uint64_t* t_ready = bars + 2;    // T diag(b) written (128 arrivals)
  uint64_t* u_done = bars + 3;
  uint64_t* t2_ready = bars + 4;   // T diag(b exp(c) kn) written
  uint64_t* w_done = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int blk = blockIdx.x, h = blockIdx.y;
  const int kh = a.tiled_heads ? (h % a.Hk) : (h / (a.Hv / a.Hk));
  const int t0 = a.blk_t0[blk], nval = a.blk_n[blk];
  const long item = long(blk) * a.Hv + h;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(ld_full, 1); mbar_init(s_done, 1); mbar_init(t_ready, 128); mbar_init(u_done, 1);
    mbar_init(t2_ready, 128); mbar_init(w_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tm_kk = tmem, tm_qk = tmem + 128, tm_u = tmem + 256, tm_w = tmem + 384;
  griddep_wait();
  griddep_launch();

  if (warp == 4) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQKV);
      mbar_expect_tx(ld_full, 6 * HALF_BYTES);
      const int q_col = kh * D, k_col = a.Hk * D + kh * D, v_col = 2 * a.Hk * D + h * D;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        tma_load_2d(q_s + hf * HALF_BYTES, &tmQKV, ld_full, q_col + hf * 64, t0);
        tma_load_2d(k_s + hf * HALF_BYTES, &tmQKV, ld_full, k_col + hf * 64, t0);
        tma_load_2d(v_s + hf * HALF_BYTES, &tmQKV, ld_full, v_col + hf * 64, t0);
      }
      bool ok = mbar_wait(ld_full, 0, abort_flag);
      if (ok) {
        tc_fence_after();
        constexpr uint32_t idesc_kk = umma_idesc(128, 128, 1, 1, 0, 0);
        const uint32_t qa = smem_u32(q_s), ka = smem_u32(k_s);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
          umma_f16(tm_kk, umma_desc_k_sw128(ka + off), umma_desc_k_sw128(ka + off), idesc_kk, k ? 1u : 0u);
          umma_f16(tm_qk, umma_desc_k_sw128(qa + off), umma_desc_k_sw128(ka + off), idesc_kk, k ? 1u : 0u);
        }
        umma_commit(s_done);
        // U = T' V, then W = T'' K: B operands are the V / K tiles read MN-major (16 token rows per step)
        constexpr uint32_t idesc_tv = umma_idesc(128, 128, 1, 1, 0, 1);
        const uint32_t ta = smem_u32(t_s), va = smem_u32(v_s);
        ok = mbar_wait(t_ready, 0, abort_flag);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t aoff = (k >> 2) * HALF_BYTES + (k & 3) * 32;
            umma_f16(tm_u, umma_desc_k_sw128(ta + aoff), umma_desc_mn_sw128(va + k * 16 * 128, HALF_BYTES, 1024), idesc_tv,
                     k ? 1u : 0u);
          }
          umma_commit(u_done);
          ok = mbar_wait(t2_ready, 0, abort_flag);
        }
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t aoff = (k >> 2) * HALF_BYTES + (k & 3) * 32;
            umma_f16(tm_w, umma_desc_k_sw128(ta + aoff), umma_desc_mn_sw128(ka + k * 16 * 128, HALF_BYTES, 1024), idesc_tv,
                     k ? 1u : 0u);
          }
          umma_commit(w_done);
        }
      }
      if (!ok) { *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_FULL); }
    }
  } else {
    // ------------------------------------------------------------------ workers: thread i = token row i of the block
    const int i = threadIdx.x;              // 0..127
    const int ch = i >> 6, il = i & 63;     // chunk of the block, row inside the chunk
    const bool valid = i < nval;
    const uint32_t lane_off = uint32_t(warp * 32) << 16;
    // zero the off-diagonal halves of T' (rows of chunk 0 in token half 1, rows of chunk 1 in token half 0)
    {
      uint4* z = reinterpret_cast<uint4*>(t_s + (ch ^ 1) * HALF_BYTES + i * 128);
#pragma unroll
      for (int c = 0; c < 8; ++c) z[c] = make_uint4(0u, 0u, 0u, 0u);
    }
    // gates: inclusive scan of g inside the chunk (two warps per chunk)
    float gv = valid ? a.g[long(t0 + i) * a.Hv + h] : 0.f;
    const float bv = valid ? a.beta[long(t0 + i) * a.Hv + h] : 0.f;
    float cs = gv;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, cs, o);
      if (lane >= o) cs += n;
    }
    if (lane == 31) cs_s[warp] = cs;        // warp totals (scratch before the real values land)
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (warp & 1) cs += cs_s[warp - 1];
    asm volatile("bar.sync 1, 128;" ::: "memory");
    cs_s[i] = cs;
    be_s[i] = bv;
    // row norms from the landed tiles
    bool ok = mbar_wait(ld_full, 0, abort_flag);
    float qq = 0.f, kk = 0.f;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      const uint4 uq = *reinterpret_cast<const uint4*>(q_s + (c >> 3) * HALF_BYTES + i * 128 + (c & 7) * 16);
      const uint4 uk = *reinterpret_cast<const uint4*>(k_s + (c >> 3) * HALF_BYTES + i * 128 + (c & 7) * 16);
      const __nv_bfloat162* pq = reinterpret_cast<const __nv_bfloat162*>(&uq);
      const __nv_bfloat162* pk = reinterpret_cast<const __nv_bfloat162*>(&uk);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 fq = __bfloat1622float2(pq[e]), fk = __bfloat1622float2(pk[e]);
        qq += fq.x * fq.x + fq.y * fq.y;
        kk += fk.x * fk.x + fk.y * fk.y;
      }
    }
    const float qn = valid ? rsqrtf(qq + a.l2_eps) * a.scale : 0.f;
    const float kn = valid ? rsqrtf(kk + a.l2_eps) : 0.f;
    qn_s[i] = qn;
    kn_s[i] = kn;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const float c_end = cs_s[ch * 64 + 63];
    if (il == 63) a.gC[item * 2 + ch] = __expf(cs);

    // ---- A (fp32 scratch) and M (global) from K K^T and Q K^T
    if (ok) ok = mbar_wait(s_done, 0, abort_flag);
    tc_fence_after();
    float* a_row = a_s + (ch * CH + il) * PREP_A_STRIDE;
    __nv_bfloat16* m_row = a.M + (item * 128 + i) * 64;
#pragma unroll 1
    for (int c0 = 0; c0 < 64; c0 += 32) {
      uint32_t rk[32], rq[32];
      tmem_ld32(tm_kk + lane_off + ch * 64 + c0, rk);
      tmem_ld32(tm_qk + lane_off + ch * 64 + c0, rq);
      tmem_ld_wait();
      uint32_t packed[16];
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        float mv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int jj = c0 + j + e;                         // column token inside the chunk
          const float dec = __expf(cs - cs_s[ch * 64 + jj]);
          const float knj = kn_s[ch * 64 + jj];
          a_row[jj] = jj < il ? bv * kn * knj * dec * __uint_as_float(rk[j + e]) : 0.f;
          mv[e] = (jj <= il && valid) ? qn * knj * dec * __uint_as_float(rq[j + e]) : 0.f;
        }
        const __nv_bfloat162 bb = __floats2bfloat162_rn(mv[0], mv[1]);
        packed[j / 2] = *reinterpret_cast<const uint32_t*>(&bb);
      }
#pragma unroll
      for (int c = 0; c < 4; ++c)
        reinterpret_cast<uint4*>(m_row + c0)[c] = make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // ---- T = (I + A)^-1 by forward substitution: this thread owns column `il` of its chunk's T
    float t[CH];
    {
      const float* A = a_s + ch * CH * PREP_A_STRIDE;
#pragma unroll
      for (int m = 0; m < CH; ++m) {
        float acc = (m == il) ? 1.f : 0.f;
#pragma unroll
        for (int l = 0; l < m; ++l) acc = fmaf(-A[m * PREP_A_STRIDE + l], t[l], acc);
        t[m] = acc;
      }
    }
    // T' = T diag(b): element (row m, column token il) of the chunk's diagonal block
    const float su = be_s[i];
    const float sw = su * __expf(cs) * kn;
#pragma unroll
    for (int m = 0; m < CH; ++m)
      *reinterpret_cast<__nv_bfloat16*>(t_s + ch * HALF_BYTES + (ch * 64 + m) * 128 + (((il >> 3) ^ (m & 7)) << 4) + ((il & 7) << 1)) =
          __float2bfloat16(t[m] * su);
    fence_proxy_async_smem();
    tc_fence_before();
    mbar_arrive(t_ready);
    // ---- scaled copies of K and Q for the scan: K' = exp(c_end - c) kn K, Q' = exp(c) qn Q (rows of this thread)
    {
      const float fk = valid ? __expf(c_end - cs) * kn : 0.f;
      const float fq = valid ? __expf(cs) * qn : 0.f;
      __nv_bfloat16* kd_row = a.Kd + (item * 128 + i) * D;
      __nv_bfloat16* qg_row = a.Qg + (item * 128 + i) * D;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const int phys = (c >> 3) * HALF_BYTES + i * 128 + (((c & 7) ^ (i & 7)) << 4);
        uint4 uk = *reinterpret_cast<const uint4*>(k_s + phys);
        uint4 uq = *reinterpret_cast<const uint4*>(q_s + phys);
        __nv_bfloat162* pk = reinterpret_cast<__nv_bfloat162*>(&uk);
        __nv_bfloat162* pq = reinterpret_cast<__nv_bfloat162*>(&uq);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f1 = __bfloat1622float2(pk[e]), f2 = __bfloat1622float2(pq[e]);
          pk[e] = __floats2bfloat162_rn(f1.x * fk, f1.y * fk);
          pq[e] = __floats2bfloat162_rn(f2.x * fq, f2.y * fq);
        }
        reinterpret_cast<uint4*>(kd_row)[c] = uk;
        reinterpret_cast<uint4*>(qg_row)[c] = uq;
      }
    }
    // ---- U out, then T'' = T diag(b exp(c) kn) over the same tile, then W out
    if (ok) ok = mbar_wait(u_done, 0, abort_flag);
    tc_fence_after();
#pragma unroll
    for (int m = 0; m < CH; ++m)
      *reinterpret_cast<__nv_bfloat16*>(t_s + ch * HALF_BYTES + (ch * 64 + m) * 128 + (((il >> 3) ^ (m & 7)) << 4) + ((il & 7) << 1)) =
          __float2bfloat16(t[m] * sw);
    fence_proxy_async_smem();
    tc_fence_before();
    mbar_arrive(t2_ready);
    auto store_rows = [&](uint32_t tm, __nv_bfloat16* dst) {
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tm + lane_off + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(r[8 * c]), __uint_as_float(r[8 * c + 1]));
          o.y = pack_bf16x2(__uint_as_float(r[8 * c + 2]), __uint_as_float(r[8 * c + 3]));
          o.z = pack_bf16x2(__uint_as_float(r[8 * c + 4]), __uint_as_float(r[8 * c + 5]));
          o.w = pack_bf16x2(__uint_as_float(r[8 * c + 6]), __uint_as_float(r[8 * c + 7]));
          reinterpret_cast<uint4*>(dst + c0)[c] = o;
        }
      }
    };
    store_rows(tm_u, a.U + (item * 128 + i) * D);
    if (ok) ok = mbar_wait(w_done, 0, abort_flag);
    tc_fence_after();
    store_rows(tm_w, a.W + (item * 128 + i) * D);
    if (!ok) { *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_FULL); }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// SCAN: grid (value heads, sequences), 160 threads: warps 0..3 = workers (thread = dv row), warp 4 = TMA + MMA.
// ---------------------------------------------------------------------------------------------------------------
struct ScanArgs {
  const int* seq_blk0; const int* seq_nchunk; const int* seq_t0; const int* seq_len; const int* slots;
  const float* gC;                 // [items * 2]
  float* state;                    // [slots, Hv, dk, dv] fp32
  __nv_bfloat16* out;              // [T, Hv, dv]
  int Hv, write_state;
  int* status;
};
constexpr int SC_W = 2 * CH * 128;      // W / Q' / K' chunk tile: two 64-column halves of 64 rows
constexpr int SC_M = CH * 128;          // M chunk tile
constexpr int SC_U = CH * D * 2;        // U chunk tile (plain rows)
constexpr int SC_STAGE = 3 * SC_W + SC_M + SC_U;          // 73728
constexpr int SC_SMEM = 2 * HALF_BYTES + HALF_BYTES + 2 * SC_STAGE + 1024 + 256;

__global__ void __launch_bounds__(160, 1)
gdn_chunk_scan_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmQg,
                      const __grid_constant__ CUtensorMap tmKd, const __grid_constant__ CUtensorMap tmM,
                      const __grid_constant__ CUtensorMap tmU, const ScanArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_a = smem;                          // S^T  [2 dk halves][128 dv rows][128 B]
  uint8_t* d_a = s_a + 2 * HALF_BYTES;          // D^T  [128 dv rows][64 tokens]
  uint8_t* stg = d_a + HALF_BYTES;              // [2] x {W, Q', K', M, U}
  uint64_t* bars = reinterpret_cast<uint64_t*>(stg + 2 * SC_STAGE);
  uint64_t* ld_full = bars;        // [2]
  uint64_t* s_ready = bars + 2;    // state operand + scaled accumulator ready (128 arrivals)
  uint64_t* d_done = bars + 3;     // W S0 and Q' S0 done
  uint64_t* dl_ready = bars + 4;   // D^T written (128 arrivals)
  uint64_t* o_done = bars + 5;     // M D and K'^T D done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int h = blockIdx.x, seq = blockIdx.y;
  const int nchunk = a.seq_nchunk[seq];
  const int blk0 = a.seq_blk0[seq];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(&ld_full[0], 1); mbar_init(&ld_full[1], 1);
    mbar_init(s_ready, 128); mbar_init(d_done, 1); mbar_init(dl_ready, 128); mbar_init(o_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tm_d = tmem, tm_o = tmem + 64, tm_s = tmem + 128;
  griddep_wait();
  griddep_launch();
  auto chunk_row = [&](int c) -> int {      // first row of chunk c in the [items * 128, .] scratch tensors
    return int((long(blk0 + (c >> 1)) * a.Hv + h) * 128 + (c & 1) * 64);
  };

  if (warp == 4) {
    if (lane == 0 && nchunk > 0) {
      tma_prefetch_desc(&tmW); tma_prefetch_desc(&tmQg); tma_prefetch_desc(&tmKd); tma_prefetch_desc(&tmM);
      tma_prefetch_desc(&tmU);
      auto load_chunk = [&](int c) {
        uint8_t* st = stg + (c & 1) * SC_STAGE;
        uint64_t* bar = &ld_full[c & 1];
        const int r0 = chunk_row(c);
        mbar_expect_tx(bar, SC_STAGE);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          tma_load_2d(st + hf * (CH * 128), &tmW, bar, hf * 64, r0);
          tma_load_2d(st + SC_W + hf * (CH * 128), &tmQg, bar, hf * 64, r0);
          tma_load_2d(st + 2 * SC_W + hf * (CH * 128), &tmKd, bar, hf * 64, r0);
        }
        tma_load_2d(st + 3 * SC_W, &tmM, bar, 0, r0);
        tma_load_2d(st + 3 * SC_W + SC_M, &tmU, bar, 0, r0);
      };
      constexpr uint32_t idesc_d = umma_idesc(128, 64, 1, 1, 0, 0);      // D^T / O^T: N = 64 tokens
      constexpr uint32_t idesc_s = umma_idesc(128, 128, 1, 1, 0, 1);     // S^T update: B = K' MN-major
      load_chunk(0);
      bool ok = true;
      for (int c = 0; ok && c < nchunk; ++c) {
        const uint32_t st = smem_u32(stg + (c & 1) * SC_STAGE);
        ok = mbar_wait(s_ready, c & 1, abort_flag);        // S operand of this chunk ready; other stage is free
        if (!ok) break;
        if (c + 1 < nchunk) load_chunk(c + 1);
        ok = mbar_wait(&ld_full[c & 1], (c >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sa = smem_u32(s_a), da = smem_u32(d_a);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t adesc = umma_desc_k_sw128(sa + (k >> 2) * HALF_BYTES + (k & 3) * 32);
          const uint32_t boff = (k >> 2) * (CH * 128) + (k & 3) * 32;
          umma_f16(tm_d, adesc, umma_desc_k_sw128(st + boff), idesc_d, k ? 1u : 0u);
          umma_f16(tm_o, adesc, umma_desc_k_sw128(st + SC_W + boff), idesc_d, k ? 1u : 0u);
        }
        umma_commit(d_done);
        ok = mbar_wait(dl_ready, c & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t adesc = umma_desc_k_sw128(da + k * 32);
          umma_f16(tm_o, adesc, umma_desc_k_sw128(st + 3 * SC_W + k * 32), idesc_d, 1u);
          umma_f16(tm_s, adesc, umma_desc_mn_sw128(st + 2 * SC_W + k * 16 * 128, CH * 128, 1024), idesc_s, 1u);
        }
        umma_commit(o_done);
      }
      if (!ok) { *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_FULL); }
    }
  } else if (nchunk > 0) {
    // ------------------------------------------------------------------ workers: thread r = dv row r
    const int r = threadIdx.x;
    const uint32_t lane_off = uint32_t(warp * 32) << 16;
    const int slot = a.slots[seq];
    float* st_g = a.state + (long(slot) * a.Hv + h) * D * D;            // [dk][dv]
    const int seq_t0 = a.seq_t0[seq], seq_len = a.seq_len[seq];
    // S^T row r from the state (column r of S), as bf16 operand and (times the first chunk's decay) as accumulator
    auto put_state = [&](const float (&v)[32], int c0, float next_decay) {
      uint32_t acc[32];
      uint32_t packed[16];
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        acc[j] = __float_as_uint(v[j] * next_decay);
        acc[j + 1] = __float_as_uint(v[j + 1] * next_decay);
        packed[j / 2] = pack_bf16x2(v[j], v[j + 1]);
      }
      tmem_st32(tm_s + lane_off + c0, acc);
      uint8_t* base = s_a + (c0 >> 6) * HALF_BYTES + r * 128;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int chunk = (((c0 & 63) >> 3) + q) ^ (r & 7);
        *reinterpret_cast<uint4*>(base + chunk * 16) =
            make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
      }
    };
    {
      const float dec0 = a.gC[(long(blk0) * a.Hv + h) * 2];
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = st_g[long(c0 + j) * D + r];
        put_state(v, c0, dec0);
      }
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(s_ready);
    }
    bool ok = true;
    for (int c = 0; c < nchunk; ++c) {
      const uint8_t* st = stg + (c & 1) * SC_STAGE;
      const __nv_bfloat16* u_s = reinterpret_cast<const __nv_bfloat16*>(st + 3 * SC_W + SC_M);   // [64 tok][128 dv]
      // ---- D^T = U^T - (W S0)^T
      if (ok) ok = mbar_wait(d_done, c & 1, abort_flag);
      tc_fence_after();
#pragma unroll 1
      for (int c0 = 0; c0 < CH; c0 += 32) {
        uint32_t rr[32];
        tmem_ld32(tm_d + lane_off + c0, rr);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float d0 = __bfloat162float(u_s[(c0 + j) * D + r]) - __uint_as_float(rr[j]);
          const float d1 = __bfloat162float(u_s[(c0 + j + 1) * D + r]) - __uint_as_float(rr[j + 1]);
          packed[j / 2] = pack_bf16x2(d0, d1);
        }
        uint8_t* base = d_a + r * 128;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = ((c0 >> 3) + q) ^ (r & 7);
          *reinterpret_cast<uint4*>(base + chunk * 16) =
              make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(dl_ready);
      // ---- outputs of the chunk and the new state
      if (ok) ok = mbar_wait(o_done, c & 1, abort_flag);
      tc_fence_after();
      const int tok0 = seq_t0 + c * CH;
      const int nt = min(CH, seq_len - c * CH);
#pragma unroll 1
      for (int c0 = 0; c0 < CH; c0 += 32) {
        uint32_t rr[32];
        tmem_ld32(tm_o + lane_off + c0, rr);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (c0 + j < nt) a.out[(long(tok0 + c0 + j) * a.Hv + h) * D + r] = __float2bfloat16(__uint_as_float(rr[j]));
      }
      const bool last = c + 1 == nchunk;
      const float dec_next = last ? 1.f : a.gC[(long(blk0 + ((c + 1) >> 1)) * a.Hv + h) * 2 + ((c + 1) & 1)];
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t rr[32];
        tmem_ld32(tm_s + lane_off + c0, rr);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(rr[j]);
        if (last) {
          if (a.write_state) {
#pragma unroll
            for (int j = 0; j < 32; ++j) st_g[long(c0 + j) * D + r] = v[j];
          }
        } else {
          put_state(v, c0, dec_next);
        }
      }
      if (!last) {
        tmem_st_wait();
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(s_ready);
      }
    }
    if (!ok) { *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_FULL); }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

}  // namespace

size_t gdn_chunk_scratch_bytes(int n_blocks, int Hv) {
  const size_t items = size_t(n_blocks) * Hv;
  return items * (4 * 128 * 128 * 2 + 128 * 64 * 2) + items * 2 * 4 + 256;
}

int gdn_chunk_launch(const void* qkv, long ld, long T, const float* g, const float* beta, float* state,
                     const int* blk_t0, const int* blk_n, int n_blocks, const int* seq_blk0, const int* seq_nchunk,
                     const int* seq_t0, const int* seq_len, const int* slots, int n_seqs, int Hk, int Hv, int DK, int DV,
                     int tiled_heads, float scale, float l2_eps, void* out, int write_state, void* scratch,
                     int* status, cudaStream_t s) {
  if (DK != 128 || DV != 128 || n_blocks <= 0 || n_seqs <= 0 || Hk <= 0 || Hv % Hk || (ld % 8) ||
      (reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(scratch) & 255))
    return 1;
  const size_t items = size_t(n_blocks) * Hv;
  auto* base = static_cast<__nv_bfloat16*>(scratch);
  PrepArgs pa{};
  pa.g = g; pa.beta = beta; pa.blk_t0 = blk_t0; pa.blk_n = blk_n; pa.Hk = Hk; pa.Hv = Hv; pa.tiled_heads = tiled_heads;
  pa.scale = scale; pa.l2_eps = l2_eps;
  pa.U = base; pa.W = pa.U + items * 128 * 128; pa.Kd = pa.W + items * 128 * 128; pa.Qg = pa.Kd + items * 128 * 128;
  pa.M = pa.Qg + items * 128 * 128;
  pa.gC = reinterpret_cast<float*>(pa.M + items * 128 * 64);
  pa.status = status;
  const long C = 2L * Hk * DK + long(Hv) * DV;
  const CUtensorMap* tmQKV = tmap_2d(qkv, uint64_t(T), uint64_t(C), uint64_t(ld) * 2, 128, 64, TM_BF16, true);
  const uint64_t rows = items * 128;
  const CUtensorMap* tmW = tmap_2d(pa.W, rows, 128, 256, 64, 64, TM_BF16, true);
  const CUtensorMap* tmQg = tmap_2d(pa.Qg, rows, 128, 256, 64, 64, TM_BF16, true);
  const CUtensorMap* tmKd = tmap_2d(pa.Kd, rows, 128, 256, 64, 64, TM_BF16, true);
  const CUtensorMap* tmM = tmap_2d(pa.M, rows, 64, 128, 64, 64, TM_BF16, true);
  const CUtensorMap* tmU = tmap_2d(pa.U, rows, 128, 256, 64, 128, TM_BF16, false);
  if (!tmQKV || !tmW || !tmQg || !tmKd || !tmM || !tmU) return 1;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(gdn_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PREP_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(gdn_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SC_SMEM) != cudaSuccess)
      return 1;
    attr = true;
  }
  launch_pdl(gdn_chunk_prep_kernel, dim3(n_blocks, Hv), dim3(160), PREP_SMEM, s, *tmQKV, pa);
  if (cudaGetLastError() != cudaSuccess) return 1;
  ScanArgs sa{};
  sa.seq_blk0 = seq_blk0; sa.seq_nchunk = seq_nchunk; sa.seq_t0 = seq_t0; sa.seq_len = seq_len; sa.slots = slots;
  sa.gC = pa.gC; sa.state = state; sa.out = static_cast<__nv_bfloat16*>(out); sa.Hv = Hv; sa.write_state = write_state;
  sa.status = status;
  launch_pdl(gdn_chunk_scan_kernel, dim3(Hv, n_seqs), dim3(160), SC_SMEM, s, *tmW, *tmQg, *tmKd, *tmM, *tmU, sa);
  return cudaGetLastError() != cudaSuccess;
}

}  // namespace lb
