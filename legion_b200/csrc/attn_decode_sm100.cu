// Paged decode attention on tcgen05 for sm_100a (flash-decoding, GQA heads share every K/V byte).
//
// One CTA = (kv head, sequence, split). The KEYS are the UMMA M dimension, so a block of 128 cached
// tokens is one 128-lane TMEM tile and the handful of query heads that share the kv head are the
// N dimension (padded to 16):
//     S^T[128 keys, 16 q] = K[128, D] . Q^T            (K tile: K-major A operand, straight from TMA)
//     O^T[D, 16 q]       += V^T[D, 128 keys] . P        (V tile: MN-major A operand, same TMA layout)
// Warps 0..3: thread t owns key t of the block (a TMEM lane of S^T) and later output dim t (a lane of
// O^T). Column maxima over the 128 keys use redux.sync on order-preserving integer images of the
// scores, row sums stay thread-local until the end, O^T is rescaled in TMEM only when a maximum moved.
// Warp 4, one lane: TMA loads of K (double buffered) and V pages through the block table and both MMAs.
// Shared memory per CTA is 2 K tiles + 1 V tile, so two CTAs fit an SM for head dim 128 and their
// dependency chains interleave. Split count is a launch constant, lengths and tables are data.
//
// Counterpart in the reference: src/cuda/paged_attn/common.cuh (paged_decode, paged_combine).
#include "common.cuh"
#include "kernels.h"
#include "tmap.cuh"

namespace lb {

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait2() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ int f2ord(float f) {
  const int i = __float_as_int(f);
  return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float ord2f(int i) { return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff); }

struct DecodeTcArgs {
  const int* ctx_lens;
  const int* block_table;
  int table_width, page;
  int Hq, Hkv, n_splits;
  float scale_log2;
  int window;
  float* o_part;   // [B, Hq, n_splits, D]
  float* ml_part;  // [B, Hq, n_splits, 2] (max in natural-log units, sum)
  int* status;
};

template <int D>
struct DecodeTcCfg {
  static constexpr int NQ = 16;
  static constexpr int BKV = 128;
  static constexpr int HALVES = D / 64;
  static constexpr int KV_BYTES = HALVES * BKV * 128;
  static constexpr int Q_BYTES = HALVES * NQ * 128;
  static constexpr int P_BYTES = 2 * NQ * 128;
  static constexpr int K_STAGES = 2;
  static constexpr int MT = D <= 128 ? 1 : D / 128;        // 128-row M tiles of O^T
  static constexpr int TMEM_COLS = (NQ + MT * NQ <= 32) ? 32 : 64;
  static constexpr int SMEM = K_STAGES * KV_BYTES + KV_BYTES + Q_BYTES + P_BYTES + 1024 + 1024;
};

template <int D>
__global__ void __launch_bounds__(160)
paged_decode_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const DecodeTcArgs a) {
  using Cfg = DecodeTcCfg<D>;
  constexpr int NQ = Cfg::NQ, BKV = Cfg::BKV, HALVES = Cfg::HALVES, MT = Cfg::MT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_s = smem;                                   // [K_STAGES]
  uint8_t* v_s = k_s + Cfg::K_STAGES * Cfg::KV_BYTES;    // single stage
  uint8_t* q_s = v_s + Cfg::KV_BYTES;
  uint8_t* p_s = q_s + Cfg::Q_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + Cfg::P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;   // [2]
  uint64_t* v_full = bars + 3;
  uint64_t* s_full = bars + 4;
  uint64_t* p_ready = bars + 5;
  uint64_t* o_done = bars + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* smax = reinterpret_cast<float*>(bars + 10);       // [NQ][4 warps], 16-byte aligned
  float* ssum = smax + NQ * 4;                             // [NQ][4]

  const int G = a.Hq / a.Hkv;
  const int gtiles = (G + NQ - 1) / NQ;
  const int kvh = blockIdx.x / gtiles;
  const int g0 = (blockIdx.x % gtiles) * NQ;
  const int gn = min(NQ, G - g0);
  const int b = blockIdx.y;
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int ctx = a.ctx_lens[b];
  const int start = (a.window > 0 && ctx > a.window) ? ctx - a.window : 0;
  const int blk_first = start / BKV;
  const int n_units = (ctx + BKV - 1) / BKV - blk_first;
  const int units_per = (n_units + a.n_splits - 1) / a.n_splits;
  const int blk_lo = blk_first + split * units_per;
  const int blk_hi = min((ctx + BKV - 1) / BKV, blk_lo + units_per);
  const int n_blk = max(0, blk_hi - blk_lo);
  const int head0 = kvh * G + g0;

  if (n_blk == 0) {  // empty split: neutral partials, no barriers or TMEM touched
    for (int i = threadIdx.x; i < gn * D; i += blockDim.x) {
      const long row = (long(b) * a.Hq + head0 + i / D) * a.n_splits + split;
      a.o_part[row * D + i % D] = 0.f;
      if (i % D == 0) { a.ml_part[row * 2] = -INFINITY; a.ml_part[row * 2 + 1] = 0.f; }
    }
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(&k_full[0], 1);
    mbar_init(&k_full[1], 1);
    mbar_init(v_full, 1);
    mbar_init(s_full, 1);
    mbar_init(p_ready, 128);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;
  const uint32_t tmem_O = tmem_base + NQ;
  const int* bt = a.block_table + long(b) * a.table_width;
  const int pages_per_blk = BKV / a.page;

  if (warp == 4) {
    if (lane == 0) {
      auto load_tile = [&](const CUtensorMap* tm, uint8_t* dst, uint64_t* bar, int blk) {
        mbar_expect_tx(bar, Cfg::KV_BYTES);
        const int tok0 = blk * BKV;
        for (int p = 0; p < pages_per_blk; ++p) {
          const int tok = tok0 + p * a.page;
          const int pg = (tok < ctx) ? bt[tok / a.page] : bt[0];
#pragma unroll
          for (int h = 0; h < HALVES; ++h)
            tma_load_3d(dst + h * (BKV * 128) + p * a.page * 128, tm, bar, h * 64, kvh, pg * a.page);
        }
      };
      mbar_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
      for (int h = 0; h < HALVES; ++h) tma_load_3d(q_s + h * (NQ * 128), &tmQ, q_full, h * 64, head0, b);
      load_tile(&tmK, k_s, &k_full[0], blk_lo);
      if (n_blk > 1) load_tile(&tmK, k_s + Cfg::KV_BYTES, &k_full[1], blk_lo + 1);
      load_tile(&tmV, v_s, v_full, blk_lo);
      constexpr uint32_t idesc_s = umma_idesc(128, NQ, 1, 1, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc(128, NQ, 1, 1, 1, 0);   // A (= V^T) is MN-major
      bool ok = mbar_wait(q_full, 0, abort_flag);
      if (!ok) { *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_FULL); }
      for (int i = 0; ok && i < n_blk; ++i) {
        const int st = i & 1;
        if (!mbar_wait(&k_full[st], (i >> 1) & 1, abort_flag)) {
          *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_FULL); break;
        }
        tc_fence_after();
        const uint32_t ka = smem_u32(k_s + st * Cfg::KV_BYTES);
        const uint32_t qa = smem_u32(q_s);
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t da = umma_desc_k_sw128(ka + h * (BKV * 128) + k * 32);
            const uint64_t db = umma_desc_k_sw128(qa + h * (NQ * 128) + k * 32);
            umma_f16(tmem_S, da, db, idesc_s, (h | k) ? 1u : 0u);
          }
        }
        umma_commit(s_full);
        if (!mbar_wait(p_ready, i & 1, abort_flag)) {
          *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_FLAG); break;
        }
        // S(i) has been consumed, so K stage st is free: prefetch block i + 2 into it
        if (i + 2 < n_blk) load_tile(&tmK, k_s + st * Cfg::KV_BYTES, &k_full[st], blk_lo + i + 2);
        if (!mbar_wait(v_full, i & 1, abort_flag)) {
          *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_FULL); break;
        }
        tc_fence_after();
        const uint32_t va = smem_u32(v_s);
        const uint32_t pa = smem_u32(p_s);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
          for (int k = 0; k < BKV / 16; ++k) {
            // A = V^T rows [mt*128, mt*128+128) of d: two 64-wide MN groups, LBO apart; D = 64 reads the
            // only group twice (LBO 0) and the duplicate lanes are never stored.
            const uint32_t lbo = (D == 64) ? 0u : uint32_t(BKV * 128);
            const uint64_t da = umma_desc_mn_sw128(va + mt * 2 * (BKV * 128) + k * 16 * 128, lbo, 1024);
            const uint64_t db = umma_desc_k_sw128(pa + (k / 4) * (NQ * 128) + (k % 4) * 32);
            umma_f16(tmem_O + mt * NQ, da, db, idesc_o, (i | k) ? 1u : 0u);
          }
        }
        umma_commit(o_done);
        // the single V stage is free once this PV has completed
        if (i + 1 < n_blk) {
          if (!mbar_wait(o_done, i & 1, abort_flag)) {
            *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_EMPTY); break;
          }
          load_tile(&tmV, v_s, v_full, blk_lo + i + 1);
        }
      }
    }
  } else {
    const int tl = warp * 32 + lane;            // key within the block, later output dim within a tile
    const uint32_t lane_off = uint32_t(warp * 32) << 16;
    float m_run[NQ], l_run[NQ];
#pragma unroll
    for (int q = 0; q < NQ; ++q) { m_run[q] = -INFINITY; l_run[q] = 0.f; }
    bool ok = true;
    for (int i = 0; i < n_blk; ++i) {
      if (!__all_sync(0xffffffffu, mbar_wait(s_full, i & 1, abort_flag))) {
        *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_FULL); ok = false; break;
      }
      tc_fence_after();
      uint32_t r[16];
      tmem_ld16(tmem_S + lane_off, r);
      tmem_ld_wait();
      const int tok = (blk_lo + i) * BKV + tl;
      const bool valid = tok >= start && tok < ctx;
      float s[NQ];
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        s[q] = valid ? __uint_as_float(r[q]) * a.scale_log2 : -INFINITY;
        const int wm = __reduce_max_sync(0xffffffffu, f2ord(s[q]));
        if (lane == q) smax[q * 4 + warp] = ord2f(wm);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      float alpha[NQ];
      bool moved = false;
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const float4 m4 = *reinterpret_cast<const float4*>(&smax[q * 4]);
        const float m_new = fmaxf(m_run[q], fmaxf(fmaxf(m4.x, m4.y), fmaxf(m4.z, m4.w)));
        alpha[q] = (m_run[q] == -INFINITY) ? 0.f : exp2f(m_run[q] - m_new);
        moved |= (m_new != m_run[q]);
        m_run[q] = m_new;
      }
      // P may be overwritten and O rescaled only after the previous PV has finished
      if (i >= 1) {
        if (!__all_sync(0xffffffffu, mbar_wait(o_done, (i - 1) & 1, abort_flag))) {
          *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_EMPTY); ok = false; break;
        }
        tc_fence_after();
      }
      // probabilities: P[q][key] bf16, K-major rows of 128 bytes per 64-key half, 128-byte swizzle
      uint8_t* prow = p_s + (tl / 64) * (NQ * 128);
      const int kc = tl % 64;
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        float p = 0.f;
        if (valid && m_run[q] != -INFINITY) p = exp2f(s[q] - m_run[q]);
        const __nv_bfloat16 pb = __float2bfloat16(p);
        l_run[q] = l_run[q] * alpha[q] + __bfloat162float(pb);
        const int chunk = (kc / 8) ^ (q & 7);
        *reinterpret_cast<__nv_bfloat16*>(prow + q * 128 + chunk * 16 + (kc % 8) * 2) = pb;
      }
      if (i >= 1 && moved) {   // uniform over the CTA: every thread sees the same maxima
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          uint32_t o[16];
          tmem_ld16(tmem_O + mt * NQ + lane_off, o);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < NQ; ++q) o[q] = __float_as_uint(__uint_as_float(o[q]) * alpha[q]);
          tmem_st16(tmem_O + mt * NQ + lane_off, o);
        }
        tmem_st_wait2();
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
    }
    if (ok) {
      if (!__all_sync(0xffffffffu, mbar_wait(o_done, (n_blk - 1) & 1, abort_flag))) {
        *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_FULL); ok = false;
      }
    }
    if (ok) {
      tc_fence_after();
      // total row sums: warp shuffle, then across the 4 warps through shared memory
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        float v = l_run[q];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == q) ssum[q * 4 + warp] = v;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t o[16];
        tmem_ld16(tmem_O + mt * NQ + lane_off, o);
        tmem_ld_wait();
        const int d = mt * 128 + tl;
        if (d < D) {
#pragma unroll
          for (int q = 0; q < NQ; ++q) {
            if (q < gn) {
              const long row = (long(b) * a.Hq + head0 + q) * a.n_splits + split;
              a.o_part[row * D + d] = __uint_as_float(o[q]);
            }
          }
        }
      }
      if (tl < gn) {
        const float4 s4 = *reinterpret_cast<const float4*>(&ssum[tl * 4]);
        const long row = (long(b) * a.Hq + head0 + tl) * a.n_splits + split;
        // every thread holds the same m_run; pick column tl without dynamic register indexing
        float mq = -INFINITY;
#pragma unroll
        for (int q = 0; q < NQ; ++q) if (q == tl) mq = m_run[q];
        a.ml_part[row * 2] = (mq == -INFINITY) ? -INFINITY : mq * 0.6931471805599453f;
        a.ml_part[row * 2 + 1] = s4.x + s4.y + s4.z + s4.w;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

namespace {
thread_local char g_dec_err[256];

template <int D>
int launch_decode_tc(const CUtensorMap* tq, const CUtensorMap* tk, const CUtensorMap* tv, const DecodeTcArgs& a,
                     dim3 grid, cudaStream_t s) {
  using Cfg = DecodeTcCfg<D>;
  auto kfn = paged_decode_tc_kernel<D>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess) {
      snprintf(g_dec_err, sizeof(g_dec_err), "decode attention: cannot set %d bytes of shared memory", Cfg::SMEM);
      return 1;
    }
    attr = true;
  }
  kfn<<<grid, 160, Cfg::SMEM, s>>>(*tq, *tk, *tv, a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(g_dec_err, sizeof(g_dec_err), "decode attention launch: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}
}  // namespace

const char* paged_decode_tc_last_error() { return g_dec_err; }

// Returns 0 on success, 1 on error, -1 when the shape is outside this kernel (caller falls back).
int paged_decode_tc_launch(const void* q, const void* k_cache, const void* v_cache, long n_cells, long cell_stride,
                           const int* block_table, int table_width, int page, const int* ctx_lens, float scale,
                           int window, int B, int Hq, int Hkv, int D, int n_splits, float* o_part, float* ml_part,
                           void* out, int* status, cudaStream_t s) {
  if (B <= 0) return 0;
  if ((D != 64 && D != 128 && D != 256) || page <= 0 || 128 % page != 0 || page % 8 != 0 || Hq % Hkv) return -1;
  const int G = Hq / Hkv;
  const int gtiles = (G + 15) / 16;
  const CUtensorMap* tq = tmap_3d(q, uint64_t(D), uint64_t(Hq), uint64_t(B), uint64_t(D) * 2, uint64_t(Hq) * D * 2, 64,
                                  16, 1, TM_BF16, true);
  const CUtensorMap* tk = tmap_3d(k_cache, uint64_t(D), uint64_t(Hkv), uint64_t(n_cells), uint64_t(D) * 2,
                                  uint64_t(cell_stride) * 2, 64, 1, uint32_t(page), TM_BF16, true);
  const CUtensorMap* tv = tmap_3d(v_cache, uint64_t(D), uint64_t(Hkv), uint64_t(n_cells), uint64_t(D) * 2,
                                  uint64_t(cell_stride) * 2, 64, 1, uint32_t(page), TM_BF16, true);
  if (!tq || !tk || !tv) {
    snprintf(g_dec_err, sizeof(g_dec_err), "decode attention: %s", tmap_last_error());
    return 1;
  }
  DecodeTcArgs a{};
  a.ctx_lens = ctx_lens; a.block_table = block_table; a.table_width = table_width; a.page = page;
  a.Hq = Hq; a.Hkv = Hkv; a.n_splits = n_splits; a.scale_log2 = scale * 1.4426950408889634f; a.window = window;
  a.o_part = o_part; a.ml_part = ml_part; a.status = status;
  dim3 grid(Hkv * gtiles, B, n_splits);
  int rc;
  if (D == 64) rc = launch_decode_tc<64>(tq, tk, tv, a, grid, s);
  else if (D == 128) rc = launch_decode_tc<128>(tq, tk, tv, a, grid, s);
  else rc = launch_decode_tc<256>(tq, tk, tv, a, grid, s);
  if (rc) return rc;
  return attn_combine_launch(o_part, ml_part, n_splits, B * Hq, D, out, s);
}

}  // namespace lb
