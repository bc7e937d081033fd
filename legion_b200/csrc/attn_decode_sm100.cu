// Paged decode attention on tcgen05 for sm_100a (flash-decoding, GQA heads share every K/V byte).
//
// One CTA = (kv head, sequence, split). The KEYS are the UMMA M dimension, so a block of 128 cached
// tokens is one 128-lane TMEM tile and the handful of query heads that share the kv head are the
// N dimension (padded to 16):
//     S^T[128 keys, 16 q] = K[128, D] . Q^T            (K tile: K-major A operand, straight from TMA)
//     O^T[D, 16 q]       += V^T[D, 128 keys] . P        (V tile: MN-major A operand, same TMA layout)
// Warps 0..3: thread t owns key t of the block (a TMEM lane of S^T) and later output dim t (a lane of
// O^T). Column maxima over the 128 keys use redux.sync on order-preserving integer images of the
// scores, row sums stay thread-local until the end, O^T is rescaled in TMEM only when a maximum grew
// by more than 2^8 (probabilities are taken relative to a slightly stale maximum otherwise).
// Two softmax warpgroups (warps 0..3 and 4..7) take alternate tiles; each is an independent flash-decoding
// stream with its own S^T buffer, P buffer, O^T accumulator, reference maxima and row sums, so the two
// per-tile dependency chains (TMEM load -> exponentials -> P -> barrier) run side by side and share only the
// K/V rings. Warp 8, one lane: both MMAs (scores two tiles ahead of the softmax that consumes them).
// Warp 9: TMA loads of K and V pages through the block table into rings of 3 + 3 stages (head dim 128),
// released by tcgen05.commit as soon as the MMAs have read them. One CTA per SM streams up to 192 KB of K/V at
// a time. Every warpgroup of every split writes one partial (2 x splits per head); the splits of a (sequence,
// kv head) group count themselves in when their partials are visible and the last one merges them into the
// output, so there is no combine launch. Split count is a launch constant, lengths and tables are data.
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
  float* o_part;   // [B, Hq, 2 * n_splits, D]   (part = split * 2 + warpgroup)
  float* ml_part;  // [B, Hq, 2 * n_splits, 2] (reference maximum in natural-log units, sum)
  __nv_bfloat16* out;   // [B, Hq, D]
  int* group_ctr;  // [B * gridDim.x] arrival counters of the splits, zero on entry, left zero on exit
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
  static constexpr int K_STAGES = D <= 64 ? 4 : (D <= 128 ? 3 : 2);
  static constexpr int V_STAGES = D <= 64 ? 4 : (D <= 128 ? 3 : 1);
  static constexpr int MT = D <= 128 ? 1 : D / 128;        // 128-row M tiles of O^T
  static constexpr int TMEM_COLS = (2 * NQ + 2 * MT * NQ <= 64) ? 64 : 128;   // S x 2 + O x 2 (MT x 16 each)
  static constexpr int SMEM = (K_STAGES + V_STAGES) * KV_BYTES + Q_BYTES + 2 * P_BYTES + 1024 + 1536;
  static_assert(2 * NQ + 2 * MT * NQ <= TMEM_COLS, "accumulators do not fit the TMEM allocation");
  static_assert(SMEM <= 227 * 1024, "shared memory budget");
};

// O^T is rescaled only when a column maximum grew by more than this (log2 units): the probabilities are then
// taken relative to a slightly stale maximum and stay below 2^8, exact in fp32 and harmless in bf16, and the
// TMEM round trip of the rescale leaves the per-tile critical path.
static constexpr float DEC_RESCALE_LOG2 = 8.f;

template <int D>
__global__ void __launch_bounds__(320, 1)
paged_decode_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const DecodeTcArgs a) {
  using Cfg = DecodeTcCfg<D>;
  constexpr int NQ = Cfg::NQ, BKV = Cfg::BKV, HALVES = Cfg::HALVES, MT = Cfg::MT;
  constexpr int KS = Cfg::K_STAGES, VS = Cfg::V_STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_s = smem;                                   // [KS]
  uint8_t* v_s = k_s + KS * Cfg::KV_BYTES;               // [VS]
  uint8_t* q_s = v_s + VS * Cfg::KV_BYTES;
  uint8_t* p_s = q_s + Cfg::Q_BYTES;                     // [2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + 2 * Cfg::P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;     // [4]
  uint64_t* k_empty = bars + 5;    // [4]
  uint64_t* v_full = bars + 9;     // [4]
  uint64_t* v_empty = bars + 13;   // [4]
  uint64_t* s_full = bars + 17;    // [2]
  uint64_t* p_ready = bars + 19;   // [2]
  uint64_t* o_done = bars + 21;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_islast = reinterpret_cast<int*>(tmem_slot + 2);
  float* smax = reinterpret_cast<float*>(bars + 32);       // [2 warpgroups][NQ][4 warps], 16-byte aligned
  float* ssum = smax + 2 * NQ * 4;                         // [2][NQ][4]

  const int G = a.Hq / a.Hkv;
  const int gtiles = (G + NQ - 1) / NQ;
  const int kvh = blockIdx.x / gtiles;
  const int g0 = (blockIdx.x % gtiles) * NQ;
  const int gn = min(NQ, G - g0);
  const int b = blockIdx.y;
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  griddep_wait();
  griddep_launch();
  const int ctx = a.ctx_lens[b];
  const int start = (a.window > 0 && ctx > a.window) ? ctx - a.window : 0;
  const int blk_first = start / BKV;
  const int n_units = (ctx + BKV - 1) / BKV - blk_first;
  const int units_per = (n_units + a.n_splits - 1) / a.n_splits;
  const int blk_lo = blk_first + split * units_per;
  const int blk_hi = min((ctx + BKV - 1) / BKV, blk_lo + units_per);
  const int n_blk = max(0, blk_hi - blk_lo);
  const int head0 = kvh * G + g0;

  if (threadIdx.x == 0) *abort_flag = 0;
  if (n_blk == 0) {  // empty split: neutral partials, no barriers or TMEM touched
    for (int i = threadIdx.x; i < 2 * gn * D; i += blockDim.x) {
      const int wgp = i / (gn * D), j = i % (gn * D);
      const long row = (long(b) * a.Hq + head0 + j / D) * (2 * a.n_splits) + split * 2 + wgp;
      a.o_part[row * D + j % D] = 0.f;
      if (j % D == 0) { a.ml_part[row * 2] = -INFINITY; a.ml_part[row * 2 + 1] = 0.f; }
    }
  } else {
    if (threadIdx.x == 0) {
      mbar_init(q_full, 1);
      for (int i = 0; i < 4; ++i) {
        mbar_init(&k_full[i], 1);
        mbar_init(&k_empty[i], 1);
        mbar_init(&v_full[i], 1);
        mbar_init(&v_empty[i], 1);
      }
      for (int i = 0; i < 2; ++i) {
        mbar_init(&s_full[i], 1);
        mbar_init(&p_ready[i], 128);
        mbar_init(&o_done[i], 1);
      }
      mbar_fence_init();
    }
    if (warp == 8) {
      tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
      tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_S = tmem_base;             // two buffers of NQ columns (one per warpgroup)
    const uint32_t tmem_O = tmem_base + 2 * NQ;    // two accumulators of MT x NQ columns
    const int* bt = a.block_table + long(b) * a.table_width;
    const int pages_per_blk = BKV / a.page;

    if (warp == 9) {
      // ---------------------------------------------------------------- TMA producer
      // The whole warp walks the tiles: the lanes fetch the next 32 block-table entries with one coalesced
      // load and hand them to lane 0 by shuffle, so no TMA issue waits on a table lookup of its own.
      const int ppb = pages_per_blk;                 // pages per 128-key tile (1 .. 16)
      const int tiles_per_fill = 32 / ppb;
      if (lane == 0) {
        mbar_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
        for (int h = 0; h < HALVES; ++h) tma_load_3d(q_s + h * (NQ * 128), &tmQ, q_full, h * 64, head0, b);
      }
      int pg_reg = 0;
      bool ok = true;
      for (int i = 0; ok && i < n_blk; ++i) {
        const int slot = i % tiles_per_fill;
        if (slot == 0) {
          const int pidx = (blk_lo + i) * ppb + lane;
          pg_reg = (long(pidx) * a.page < ctx) ? bt[pidx] : bt[0];
        }
        const int ks = i % KS, vs = i % VS;
        for (int kv = 0; ok && kv < 2; ++kv) {
          const int st = kv ? vs : ks, nst = kv ? VS : KS;
          uint64_t* empty = kv ? &v_empty[st] : &k_empty[st];
          uint64_t* full = kv ? &v_full[st] : &k_full[st];
          if (i >= nst && !__all_sync(0xffffffffu, mbar_wait(empty, ((i / nst) - 1) & 1, abort_flag))) {
            if (lane == 0) { *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_EMPTY); }
            ok = false;
            break;
          }
          uint8_t* dst = (kv ? v_s : k_s) + st * Cfg::KV_BYTES;
          if (lane == 0) mbar_expect_tx(full, Cfg::KV_BYTES);
          for (int p = 0; p < ppb; ++p) {
            const int pg = __shfl_sync(0xffffffffu, pg_reg, slot * ppb + p);
            if (lane == 0) {
#pragma unroll
              for (int h = 0; h < HALVES; ++h)
                tma_load_3d(dst + h * (BKV * 128) + p * a.page * 128, kv ? &tmV : &tmK, full, h * 64, kvh,
                            pg * a.page);
            }
          }
        }
      }
    } else if (warp == 8) {
      // ---------------------------------------------------------------- MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc_s = umma_idesc(128, NQ, 1, 1, 0, 0);
        constexpr uint32_t idesc_o = umma_idesc(128, NQ, 1, 1, 1, 0);   // A (= V^T) is MN-major
        const uint32_t qa = smem_u32(q_s);
        auto issue_s = [&](int i) -> bool {
          const int ks = i % KS;
          if (!mbar_wait(&k_full[ks], (i / KS) & 1, abort_flag)) return false;
          tc_fence_after();
          const uint32_t ka = smem_u32(k_s + ks * Cfg::KV_BYTES);
#pragma unroll
          for (int h = 0; h < HALVES; ++h) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint64_t da = umma_desc_k_sw128(ka + h * (BKV * 128) + k * 32);
              const uint64_t db = umma_desc_k_sw128(qa + h * (NQ * 128) + k * 32);
              umma_f16(tmem_S + (i & 1) * NQ, da, db, idesc_s, (h | k) ? 1u : 0u);
            }
          }
          umma_commit(&s_full[i & 1]);
          umma_commit(&k_empty[ks]);     // the K stage is free once these MMAs have read it
          return true;
        };
        bool ok = mbar_wait(q_full, 0, abort_flag);
        ok = ok && issue_s(0);
        if (ok && n_blk > 1) ok = issue_s(1);
        if (!ok) { *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_FULL); }
        for (int i = 0; ok && i < n_blk; ++i) {
          const int wgp = i & 1;
          if (!mbar_wait(&p_ready[wgp], (i >> 1) & 1, abort_flag)) {
            *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_FLAG); break;
          }
          const int vs = i % VS;
          if (!mbar_wait(&v_full[vs], (i / VS) & 1, abort_flag)) {
            *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_FULL); break;
          }
          tc_fence_after();
          const uint32_t va = smem_u32(v_s + vs * Cfg::KV_BYTES);
          const uint32_t pa = smem_u32(p_s + wgp * Cfg::P_BYTES);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
            for (int k = 0; k < BKV / 16; ++k) {
              // A = V^T rows [mt*128, mt*128+128) of d: two 64-wide MN groups, LBO apart; D = 64 reads the
              // only group twice (LBO 0) and the duplicate lanes are never stored.
              const uint32_t lbo = (D == 64) ? 0u : uint32_t(BKV * 128);
              const uint64_t da = umma_desc_mn_sw128(va + mt * 2 * (BKV * 128) + k * 16 * 128, lbo, 1024);
              const uint64_t db = umma_desc_k_sw128(pa + (k / 4) * (NQ * 128) + (k % 4) * 32);
              umma_f16(tmem_O + (wgp * MT + mt) * NQ, da, db, idesc_o, ((i >> 1) | k) ? 1u : 0u);
            }
          }
          umma_commit(&o_done[wgp]);
          umma_commit(&v_empty[vs]);
          // the softmax of tile i has read S[wgp]: the scores of tile i+2 go there, two tiles ahead of their use
          if (i + 2 < n_blk && !issue_s(i + 2)) {
            *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_FULL); break;
          }
        }
      }
    } else {
      // ---------------------------------------------------------------- softmax + epilogue (warps 0..7)
      const int wgp = warp >> 2;                   // warpgroup: tiles wgp, wgp + 2, ...
      const int wq = warp & 3;                     // TMEM lane quarter of this warp
      const int tl = wq * 32 + lane;               // key within the block, later output dim within a tile
      const uint32_t lane_off = uint32_t(wq * 32) << 16;
      const uint32_t my_S = tmem_S + wgp * NQ + lane_off;
      const uint32_t my_O = tmem_O + wgp * MT * NQ + lane_off;
      const int bar_id = 1 + wgp;
      float* smx = smax + wgp * (NQ * 4);
      float* ssm = ssum + wgp * (NQ * 4);
      uint8_t* my_p = p_s + wgp * Cfg::P_BYTES;
      float m_ref[NQ], l_run[NQ];
#pragma unroll
      for (int q = 0; q < NQ; ++q) { m_ref[q] = -INFINITY; l_run[q] = 0.f; }
      // rows of the padded heads are never written again: zero the P buffer once (finite B operand)
      for (int j = tl; j < Cfg::P_BYTES / 16; j += 128) reinterpret_cast<uint4*>(my_p)[j] = make_uint4(0u, 0u, 0u, 0u);
      fence_proxy_async_smem();
      // A wait that runs out does not leave the loop: the warp keeps taking part in the named barriers and the
      // p_ready arrivals (without touching TMEM or waiting again), so the other warps can never be left behind.
      bool ok = true;
      auto fail = [&](int code) { *abort_flag = 1; atomicCAS(a.status, 0, code); ok = false; };
      int n_mine = 0;
      for (int i = wgp; i < n_blk; i += 2, ++n_mine) {
        const uint32_t ph = (i >> 1) & 1;
        if (ok && !__all_sync(0xffffffffu, mbar_wait(&s_full[wgp], ph, abort_flag))) fail(ST_TIMEOUT_TMEM_FULL);
        uint32_t r[16];
#pragma unroll
        for (int q = 0; q < 16; ++q) r[q] = 0u;
        if (ok) {
          tc_fence_after();
          tmem_ld16(my_S, r);
          tmem_ld_wait();
        }
        const int tok = (blk_lo + i) * BKV + tl;
        const bool valid = tok >= start && tok < ctx;
        // Only the gn real heads are processed (the MMA's N is padded to 16). The common case needs no column
        // maxima at all: as long as no score exceeds its column's reference maximum by more than the rescale
        // threshold, the probabilities are taken relative to the (stale) reference. The "any score over"
        // vote of the 128 threads rides on the named barrier itself (bar.red.or).
        float s[NQ];
        bool over = false;
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          s[q] = -INFINITY;
          if (q < gn) {
            s[q] = valid ? __uint_as_float(r[q]) * a.scale_log2 : -INFINITY;
            over |= s[q] > m_ref[q] + DEC_RESCALE_LOG2;
          }
        }
        uint32_t any_over;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.or.pred q, %2, 128, p;\n\t"
            "selp.u32 %0, 1, 0, q;\n\t}"
            : "=r"(any_over) : "r"(over ? 1u : 0u), "r"(bar_id) : "memory");
        const bool rescale = any_over != 0;          // uniform over the warpgroup
        // this warpgroup's previous PV (tile i-2) must be done: it read the P buffer and wrote O^T
        if (ok && n_mine >= 1 && !__all_sync(0xffffffffu, mbar_wait(&o_done[wgp], ((i - 2) >> 1) & 1, abort_flag)))
          fail(ST_TIMEOUT_TMEM_EMPTY);
        if (rescale) {
          float alpha[NQ];
#pragma unroll
          for (int q = 0; q < NQ; ++q) {
            if (q < gn) {
              const int wm = __reduce_max_sync(0xffffffffu, f2ord(s[q]));
              if (lane == q) smx[q * 4 + wq] = ord2f(wm);
            }
          }
          asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
#pragma unroll
          for (int q = 0; q < NQ; ++q) {
            alpha[q] = 1.f;
            if (q < gn) {
              const float4 m4 = *reinterpret_cast<const float4*>(&smx[q * 4]);
              const float m_tile = fmaxf(fmaxf(m4.x, m4.y), fmaxf(m4.z, m4.w));
              if (m_tile > m_ref[q]) {
                alpha[q] = (m_ref[q] == -INFINITY) ? 0.f : exp2f(m_ref[q] - m_tile);
                m_ref[q] = m_tile;
              }
              l_run[q] *= alpha[q];
            }
          }
          if (ok && n_mine >= 1) {
            tc_fence_after();
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              uint32_t o[16];
              tmem_ld16(my_O + mt * NQ, o);
              tmem_ld_wait();
#pragma unroll
              for (int q = 0; q < NQ; ++q) o[q] = __float_as_uint(__uint_as_float(o[q]) * alpha[q]);
              tmem_st16(my_O + mt * NQ, o);
            }
            tmem_st_wait2();
          }
        }
        // probabilities: P[q][key] bf16, K-major rows of 128 bytes per 64-key half, 128-byte swizzle
        uint8_t* prow = my_p + (tl / 64) * (NQ * 128);
        const int kc = tl % 64;
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          if (q < gn) {
            float p = 0.f;
            if (valid && m_ref[q] != -INFINITY) p = exp2f(s[q] - m_ref[q]);
            const __nv_bfloat16 pb = __float2bfloat16(p);
            l_run[q] += __bfloat162float(pb);
            const int chunk = (kc / 8) ^ (q & 7);
            *reinterpret_cast<__nv_bfloat16*>(prow + q * 128 + chunk * 16 + (kc % 8) * 2) = pb;
          }
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(&p_ready[wgp]);
      }
      if (ok && n_mine >= 1) {
        const int last = wgp + 2 * (n_mine - 1);
        if (!__all_sync(0xffffffffu, mbar_wait(&o_done[wgp], (last >> 1) & 1, abort_flag))) fail(ST_TIMEOUT_TMEM_FULL);
      }
      // total row sums: warp shuffle, then across the 4 warps through shared memory
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        float v = l_run[q];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == q) ssm[q * 4 + wq] = v;
      }
      asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
      if (ok) {
        const int part = split * 2 + wgp, n_parts = 2 * a.n_splits;
        tc_fence_after();
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          uint32_t o[16];
#pragma unroll
          for (int q = 0; q < 16; ++q) o[q] = 0u;
          if (n_mine >= 1) {
            tmem_ld16(my_O + mt * NQ, o);
            tmem_ld_wait();
          }
          const int d = mt * 128 + tl;
          if (d < D) {
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
              if (q < gn) {
                const long row = (long(b) * a.Hq + head0 + q) * n_parts + part;
                a.o_part[row * D + d] = __uint_as_float(o[q]);
              }
            }
          }
        }
        if (tl < gn) {
          const float4 s4 = *reinterpret_cast<const float4*>(&ssm[tl * 4]);
          const long row = (long(b) * a.Hq + head0 + tl) * n_parts + part;
          // every thread holds the same m_ref; pick column tl without dynamic register indexing
          float mq = -INFINITY;
#pragma unroll
          for (int q = 0; q < NQ; ++q) if (q == tl) mq = m_ref[q];
          a.ml_part[row * 2] = (mq == -INFINITY) ? -INFINITY : mq * 0.6931471805599453f;
          a.ml_part[row * 2 + 1] = s4.x + s4.y + s4.z + s4.w;
        }
      }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
      tc_fence_after();
      tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
  }

  // ------------------------------------------------------------------ split combine by the last arriver
  // Every split CTA of a (sequence, kv head, head tile) group counts itself in after its partials are visible;
  // the last one merges the group's partials into the output, so no separate combine launch is needed.
  __threadfence();
  __syncthreads();
  const int grp = b * gridDim.x + blockIdx.x;
  if (threadIdx.x == 0) {
    const int old = atomicAdd(&a.group_ctr[grp], 1);
    *s_islast = (old == a.n_splits - 1);
    if (old == a.n_splits - 1) a.group_ctr[grp] = 0;
  }
  __syncthreads();
  if (!*s_islast || *abort_flag) return;
  __threadfence();
  // scratch in the (now idle) K stage memory: weights of every (head, split) and the heads' denominators
  float* s_w = reinterpret_cast<float*>(k_s);          // [gn][parts]
  const int ns = 2 * a.n_splits;                       // parts per head: (split, warpgroup)
  float* s_l = s_w + NQ * 256;                         // [gn]
  for (int idx = threadIdx.x; idx < gn * ns; idx += blockDim.x) {
    const long row = (long(b) * a.Hq + head0 + idx / ns) * ns + idx % ns;
    s_w[idx] = __ldcg(&a.ml_part[row * 2]);
  }
  __syncthreads();
  for (int q = warp; q < gn; q += 10) {
    float mm = -INFINITY;
    for (int sidx = lane; sidx < ns; sidx += 32) mm = fmaxf(mm, s_w[q * ns + sidx]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
    float ll = 0.f;
    for (int sidx = lane; sidx < ns; sidx += 32) {
      const float m = s_w[q * ns + sidx];
      const long row = (long(b) * a.Hq + head0 + q) * ns + sidx;
      const float wgt = (m == -INFINITY) ? 0.f : __expf(m - mm);
      ll += wgt * __ldcg(&a.ml_part[row * 2 + 1]);
      s_w[q * ns + sidx] = wgt;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ll += __shfl_xor_sync(0xffffffffu, ll, o);
    if (lane == 0) s_l[q] = ll;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < gn * D; idx += blockDim.x) {
    const int q = idx / D, d = idx % D;
    const long row0 = (long(b) * a.Hq + head0 + q) * ns;
    float o = 0.f;
    for (int sidx = 0; sidx < ns; ++sidx) {
      const float wgt = s_w[q * ns + sidx];
      if (wgt != 0.f) o += wgt * __ldcg(&a.o_part[(row0 + sidx) * D + d]);
    }
    const float ll = s_l[q];
    a.out[(long(b) * a.Hq + head0 + q) * D + d] = __float2bfloat16(ll > 0.f ? o / ll : 0.f);
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
  launch_pdl(kfn, grid, dim3(320), Cfg::SMEM, s, *tq, *tk, *tv, a);
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
                           void* out, int* group_ctr, int n_group_ctr, int* status, cudaStream_t s) {
  if (B <= 0) return 0;
  if ((D != 64 && D != 128 && D != 256) || page <= 0 || 128 % page != 0 || page % 8 != 0 || Hq % Hkv) return -1;
  const int G = Hq / Hkv;
  const int gtiles = (G + 15) / 16;
  if (n_splits < 1 || n_splits > 128 || long(B) * Hkv * gtiles > n_group_ctr) return -1;
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
  a.out = static_cast<__nv_bfloat16*>(out); a.group_ctr = group_ctr;
  dim3 grid(Hkv * gtiles, B, n_splits);
  int rc;
  if (D == 64) rc = launch_decode_tc<64>(tq, tk, tv, a, grid, s);
  else if (D == 128) rc = launch_decode_tc<128>(tq, tk, tv, a, grid, s);
  else rc = launch_decode_tc<256>(tq, tk, tv, a, grid, s);
  return rc;
}

}  // namespace lb
