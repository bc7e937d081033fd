// Paged prefill / verify attention on tcgen05 for sm_100a.
//
// One CTA = 128 query rows of one (sequence, query head). Per block of BKV keys:
//   thread X (warp 4, one lane): TMA-loads K and V pages through the block table (3-D tensor map over
//       the cache, one box per page and 64-column half, 128-byte swizzle), issues S = Q K^T into
//       TMEM, later O += P V (V is the MN-major B operand, read in place from the same smem tile)
//   warps 0..3 (thread = query row = TMEM lane): tcgen05.ld S, causal / window mask, online softmax
//       in base 2, P written back INTO tensor memory over the scores it came from (bf16 pairs, tcgen05.st) and
//       read from there as the A operand of the second MMA (no shared-memory round trip, no proxy fence), O
//       rescaled in TMEM (tcgen05.ld / st) when the running maximum moved.
// The scores are double buffered in TMEM and issued one block AHEAD: while the softmax warps work on S(i), the
// tensor pipe already computes S(i+1) (and the previous block's P V), so the softmax of block i+1 starts the moment
// block i's is done instead of waiting for P V(i) and S(i+1) to run back to back. Three K stages keep the key tile
// of block i+2 in flight, two V stages the value tile of block i+1. Head dim 128 runs with 64-key blocks: 112 KB of
// shared memory and 256 TMEM columns per CTA, so two CTAs share an SM and fill each other's remaining gaps. The softmax keeps the 64 scores of a row in registers (one TMEM read), skips the mask
// comparisons on blocks that are entirely visible, and rescales O only when the row maximum grew by more than
// 2^8 (probabilities are then relative to a slightly stale maximum).
// Sequence lengths, query offsets and block tables are data; the grid is (q tiles, heads, seqs).
//
// Counterparts in the reference: src/cuda/sm80/paged_attn.cuh (paged_prefill_mma, split verify),
// src/cuda/sm90/paged_attn_wgmma.cu.
#include "common.cuh"
#include "kernels.h"
#include "tmap.cuh"

namespace lb {

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
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// D += A B with the A operand (the probabilities, bf16 pairs in 32-bit cells, row = lane) read from tensor memory
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Packed fp32 pairs (two lanes of one 64-bit register) and the three-input maximum: the softmax of an interior block
// is bound by instruction issue (two warps per scheduler next to the tensor pipe), and these halve the scale /
// subtract, sum and maximum instructions of a row.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

struct PrefillArgs {
  const int* cu_q;         // [n_seqs + 1] first query row of each sequence
  const int* ctx_lens;     // [n_seqs] keys visible after this chunk (cached + chunk)
  const int* block_table;  // [n_seqs, table_width]
  int table_width, page;
  int Hq, Hkv;
  float scale_log2;        // softmax scale * log2(e)
  int window;              // 0 = none
  int causal;
  __nv_bfloat16* out;      // [T, Hq, D]
  int* status;
};

static constexpr float PREFILL_RESCALE_LOG2 = 8.f;

template <int D, int BKV>
struct PrefillCfg {
  static constexpr bool VSINGLE = false;
  static constexpr int HALVES = D / 64;               // 64-column (128-byte) halves of a head row
  static constexpr int Q_BYTES = HALVES * 128 * 128;  // 128 rows x 128 B per half
  static constexpr int KV_BYTES = HALVES * BKV * 128;
  static constexpr int P_BYTES = (BKV / 64) * 128 * 128;
  static constexpr int STAGES = 3;                      // K stages
  static constexpr int VSTAGES = 2;
  // no alignment slack: the dynamic shared memory of this kernel starts 1024-byte aligned (checked at entry)
  static constexpr int SMEM = Q_BYTES + (STAGES + VSTAGES) * KV_BYTES + 256;
  static constexpr int TMEM_RAW = 2 * BKV + D;          // two score buffers + the output accumulator
  static constexpr int TMEM_COLS = TMEM_RAW <= 128 ? 128 : (TMEM_RAW <= 256 ? 256 : 512);
};

template <int D, int BKV>
__global__ void __launch_bounds__(160, (D == 128 && BKV == 64) ? 2 : 1)
prefill_attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const PrefillArgs a) {
  using Cfg = PrefillCfg<D, BKV>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem_raw) & 1023u) {       // swizzled tiles need 1024-byte alignment; uniform per CTA, before any barrier
    if (threadIdx.x == 0) atomicCAS(a.status, 0, ST_BAD_ARGS);
    return;
  }
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + Cfg::Q_BYTES;                       // [STAGES] K tiles
  uint8_t* v_s = k_s + Cfg::STAGES * Cfg::KV_BYTES;        // [VSTAGES] V tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + Cfg::VSTAGES * Cfg::KV_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;   // [3]
  uint64_t* v_full = bars + 4;   // [2]
  uint64_t* s_full = bars + 6;   // [2] one per score buffer
  uint64_t* p_ready = bars + 8;  // [2] one per score buffer: with the scores issued a block ahead, a fast softmax warp
                                 //     can finish block i + 1 before a slow one has finished block i; on ONE barrier its
                                 //     second arrival would complete block i's phase early
  uint64_t* o_done = bars + 10;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int seq = blockIdx.z;
  const int head = blockIdx.y;
  const int q0 = a.cu_q[seq];
  const int q_len = a.cu_q[seq + 1] - q0;
  // causal prompts: the last query tile of a sequence has the most key blocks; tiles are handed out from the last
  // to the first so that the long ones start first and the short ones fill the tail of the grid
  const int tile_row0 = (int(gridDim.x) - 1 - int(blockIdx.x)) * 128;
  if (tile_row0 >= q_len) return;  // uniform per CTA, before any barrier or TMEM use
  const int ctx = a.ctx_lens[seq];
  const int kvh = head / (a.Hq / a.Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 3; ++i) mbar_init(&k_full[i], 1);
    mbar_init(&v_full[0], 1);
    mbar_init(&v_full[1], 1);
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(&p_ready[0], 128);
    mbar_init(&p_ready[1], 128);
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
  const uint32_t tmem_S = tmem_base;                 // score buffers at +0 and +BKV
  const uint32_t tmem_O = tmem_base + 2 * BKV;

  // key range visible to this query tile
  const int pos0 = ctx - q_len + tile_row0;                       // absolute position of tile row 0
  const int rows_here = min(128, q_len - tile_row0);
  const int last_pos = pos0 + rows_here - 1;
  const int kv_hi = a.causal ? min(ctx, last_pos + 1) : ctx;      // exclusive
  int kv_lo = 0;
  if (a.window > 0) kv_lo = max(0, pos0 - a.window + 1);
  const int blk_lo = kv_lo / BKV;
  const int blk_hi = (kv_hi + BKV - 1) / BKV;                     // exclusive
  const int n_blk = blk_hi - blk_lo;
  const int* bt = a.block_table + long(seq) * a.table_width;
  const int pages_per_blk = BKV / a.page;

  if (warp == 4) {
    if (lane == 0) {
      // ------------------------------------------------------------ loads + MMA issue
      auto load_tile = [&](const CUtensorMap* tm, uint8_t* dst, uint64_t* bar, int blk) {
        const int tok0 = blk * BKV;
        mbar_expect_tx(bar, Cfg::KV_BYTES);
        for (int p = 0; p < pages_per_blk; ++p) {
          const int tok = tok0 + p * a.page;
          // pages past the end of the sequence read cell row 0 of a valid page: masked later
          const int pg = (tok < ctx) ? bt[tok / a.page] : bt[0];
          const int cell = pg * a.page;
#pragma unroll
          for (int h = 0; h < Cfg::HALVES; ++h)
            tma_load_3d(dst + h * (BKV * 128) + p * a.page * 128, tm, bar, h * 64, kvh, cell);
        }
      };
      auto load_k = [&](int blk, int stage) { load_tile(&tmK, k_s + stage * Cfg::KV_BYTES, &k_full[stage], blk); };
      auto load_v = [&](int blk, int stage) { load_tile(&tmV, v_s + stage * Cfg::KV_BYTES, &v_full[stage], blk); };
      mbar_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
      for (int h = 0; h < Cfg::HALVES; ++h)
        tma_load_3d(q_s + h * (128 * 128), &tmQ, q_full, h * 64, head, q0 + tile_row0);
      load_k(blk_lo, 0);
      if (n_blk > 1) load_k(blk_lo + 1, 1);
      load_v(blk_lo, 0);
      if (n_blk > 1) load_v(blk_lo + 1, 1);
      constexpr uint32_t idesc_s = umma_idesc(128, BKV, 1, 1, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc(128, D, 1, 1, 0, 1);  // B (= V) is MN-major
      bool ok = mbar_wait(q_full, 0, abort_flag);
      if (!ok) { *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_FULL); }
      const uint32_t qa = smem_u32(q_s);
      // S(j) = Q K_j^T into score buffer j & 1, from K stage j % 3
      auto issue_s = [&](int j) -> bool {
        const int st = j % 3;
        if (!mbar_wait(&k_full[st], uint32_t(j / 3) & 1u, abort_flag)) {
          *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_FULL); return false;
        }
        tc_fence_after();
        const uint32_t ka = smem_u32(k_s + st * Cfg::KV_BYTES);
        const uint32_t ts = tmem_S + uint32_t(j & 1) * BKV;
#pragma unroll
        for (int h = 0; h < Cfg::HALVES; ++h) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t da = umma_desc_k_sw128(qa + h * (128 * 128) + k * 32);
            const uint64_t db = umma_desc_k_sw128(ka + h * (BKV * 128) + k * 32);
            umma_f16(ts, da, db, idesc_s, (h | k) ? 1u : 0u);
          }
        }
        umma_commit(&s_full[j & 1]);
        return true;
      };
      if (ok && n_blk > 0) ok = issue_s(0);
      for (int i = 0; ok && i < n_blk; ++i) {
        // K stage (i + 2) % 3 held block i - 1, whose scores the softmax has consumed (p_ready(i - 1) was seen)
        if (i + 2 < n_blk) load_k(blk_lo + i + 2, (i + 2) % 3);
        // the next block's scores, one block ahead of the softmax: buffer (i + 1) & 1 held S(i - 1), read and done
        if (i + 1 < n_blk && !issue_s(i + 1)) break;
        if (i >= 1 && i + 1 < n_blk) {
          // V stage (i + 1) & 1 held block i - 1: free once that block's P V has completed
          if (!mbar_wait(o_done, (i - 1) & 1, abort_flag)) {
            *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_EMPTY); break;
          }
          load_v(blk_lo + i + 1, (i + 1) & 1);
        }
        if (!mbar_wait(&p_ready[i & 1], uint32_t(i >> 1) & 1u, abort_flag)) {
          *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_FLAG); break;
        }
        if (!mbar_wait(&v_full[i & 1], uint32_t(i >> 1) & 1u, abort_flag)) {
          *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_FULL); break;
        }
        tc_fence_after();
        const uint32_t va = smem_u32(v_s + (i & 1) * Cfg::KV_BYTES);
        const uint32_t tp = tmem_S + uint32_t(i & 1) * BKV;      // P(i) sits over the scores it was computed from
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          // A = P from tensor memory: 16 keys = 8 cells of bf16 pairs per step; B = V: 16 rows of 128 B per step
          const uint64_t db = umma_desc_mn_sw128(va + k * 16 * 128, BKV * 128, 1024);
          umma_f16_ts(tmem_O, tp + k * 8, db, idesc_o, (i | k) ? 1u : 0u);
        }
        umma_commit(o_done);
      }
    }
  } else {
    // -------------------------------------------------------------- softmax warps (thread = row)
    const int row = warp * 32 + lane;
    const int qpos = pos0 + row;
    const bool row_ok = row < rows_here;
    const uint32_t lane_off = uint32_t(warp * 32) << 16;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int i = 0; i < n_blk; ++i) {
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[i & 1], uint32_t(i >> 1) & 1u, abort_flag))) {
        *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_FULL); ok = false; break;
      }
      tc_fence_after();
      const uint32_t tmem_Si = tmem_S + uint32_t(i & 1) * BKV;
      const int key0 = (blk_lo + i) * BKV;
      int hi = a.causal ? min(ctx, qpos + 1) : ctx;   // exclusive key bound for this row
      int lo = (a.window > 0) ? max(0, qpos - a.window + 1) : 0;
      if (!row_ok) { hi = 0; lo = 0; }
      // blocks entirely inside every row's visible range need no per-element mask (all interior blocks of a
      // causal prompt): uniform over the CTA
      const bool full_blk = a.window == 0 && rows_here == 128 && key0 + BKV <= (a.causal ? min(ctx, pos0 + 1) : ctx);
      float alpha = 1.f;
      float sum = 0.f;
      if (BKV <= 64) {
        // ---- one TMEM read: the row's scores stay in registers between the maximum and the exponentials
        uint32_t r[BKV <= 64 ? BKV : 1];
#pragma unroll
        for (int c = 0; c < BKV; c += 32) tmem_ld32(tmem_Si + lane_off + c, *reinterpret_cast<uint32_t(*)[32]>(&r[c]));
        tmem_ld_wait();
        float mx = -INFINITY;
        if (full_blk) {
          // four independent chains: a single one is 64 dependent operations with only two warps per scheduler
          // to hide their latency
          float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
          for (int j = 0; j < BKV; j += 8) {
            m0 = fmax3(m0, __uint_as_float(r[j]), __uint_as_float(r[j + 1]));
            m1 = fmax3(m1, __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            m2 = fmax3(m2, __uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
            m3 = fmax3(m3, __uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
          }
          mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        } else {
#pragma unroll
          for (int j = 0; j < BKV; ++j) {
            const int key = key0 + j;
            if (key >= lo && key < hi) mx = fmaxf(mx, __uint_as_float(r[j]));
          }
        }
        const float m_blk = mx * a.scale_log2;
        if (m_blk > m + PREFILL_RESCALE_LOG2 || (m == -INFINITY && m_blk != -INFINITY)) {
          alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_blk);
          m = m_blk;
        }
        const float neg_m = (m == -INFINITY) ? 0.f : -m;
        uint32_t packed[BKV <= 64 ? BKV / 2 : 1];
        if (full_blk) {
          // interior block: no mask; the row sum is taken over the fp32 probabilities in four partial sums (the
          // tensor core sees their bf16 roundings: the difference averages out far below bf16 resolution)
          const uint64_t sc2 = f2_pack(a.scale_log2, a.scale_log2), nm2 = f2_pack(neg_m, neg_m);
          uint64_t acc0 = f2_pack(0.f, 0.f), acc1 = acc0;
#pragma unroll
          for (int j = 0; j < BKV; j += 4) {
            float x0, x1, x2, x3;
            f2_unpack(f2_fma(f2_pack(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), sc2, nm2), x0, x1);
            f2_unpack(f2_fma(f2_pack(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])), sc2, nm2), x2, x3);
            const float p0 = exp2f(x0), p1 = exp2f(x1), p2 = exp2f(x2), p3 = exp2f(x3);
            acc0 = f2_add(acc0, f2_pack(p0, p1));
            acc1 = f2_add(acc1, f2_pack(p2, p3));
            packed[j / 2] = pack_bf16x2(p0, p1);
            packed[j / 2 + 1] = pack_bf16x2(p2, p3);
          }
          float s0, s1, s2, s3;
          f2_unpack(acc0, s0, s1);
          f2_unpack(acc1, s2, s3);
          sum = (s0 + s1) + (s2 + s3);
        } else {
#pragma unroll
          for (int j = 0; j < BKV; j += 2) {
            float p0 = exp2f(fmaf(__uint_as_float(r[j]), a.scale_log2, neg_m));
            float p1 = exp2f(fmaf(__uint_as_float(r[j + 1]), a.scale_log2, neg_m));
            const int key = key0 + j;
            if (!(key >= lo && key < hi)) p0 = 0.f;
            if (!(key + 1 >= lo && key + 1 < hi)) p1 = 0.f;
            // sum what the tensor core will see (bf16-rounded) to keep numerator and denominator consistent
            const __nv_bfloat162 bb = __floats2bfloat162_rn(p0, p1);
            const float2 f = __bfloat1622float2(bb);
            sum += f.x + f.y;
            packed[j / 2] = *reinterpret_cast<const uint32_t*>(&bb);
          }
        }
        // P over the scores it came from: cell c of the row holds keys 2c (low half) and 2c + 1
#pragma unroll
        for (int c = 0; c < BKV / 2; c += 16) tmem_st16(tmem_Si + lane_off + c, &packed[c]);
      } else {
        // ---- two TMEM passes (128-key blocks): row maximum, then probabilities -> swizzled smem
        float mx = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < BKV; c += 32) {
          uint32_t r[32];
          tmem_ld32(tmem_Si + lane_off + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int key = key0 + c + j;
            if (full_blk || (key >= lo && key < hi)) mx = fmaxf(mx, __uint_as_float(r[j]));
          }
        }
        const float m_blk = mx * a.scale_log2;
        if (m_blk > m + PREFILL_RESCALE_LOG2 || (m == -INFINITY && m_blk != -INFINITY)) {
          alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_blk);
          m = m_blk;
        }
        const float neg_m = (m == -INFINITY) ? 0.f : -m;
#pragma unroll 1
        for (int c = 0; c < BKV; c += 32) {
          uint32_t r[32];
          tmem_ld32(tmem_Si + lane_off + c, r);
          tmem_ld_wait();
          uint32_t packed[16];
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float p0 = exp2f(fmaf(__uint_as_float(r[j]), a.scale_log2, neg_m));
            float p1 = exp2f(fmaf(__uint_as_float(r[j + 1]), a.scale_log2, neg_m));
            const int key = key0 + c + j;
            if (!full_blk && !(key >= lo && key < hi)) p0 = 0.f;
            if (!full_blk && !(key + 1 >= lo && key + 1 < hi)) p1 = 0.f;
            const __nv_bfloat162 bb = __floats2bfloat162_rn(p0, p1);
            const float2 f = __bfloat1622float2(bb);
            sum += f.x + f.y;
            packed[j / 2] = *reinterpret_cast<const uint32_t*>(&bb);
          }
          // in place: the 32 score cells just read become 16 cells of bf16 pairs at half the column offset
          // (cells below c / 2 + 16 <= c were read by earlier chunks of this thread)
          tmem_st16(tmem_Si + lane_off + c / 2, packed);
        }
      }
      l = l * alpha + sum;
      if (i >= 1) {
        // every thread rescales its own O row; with the lazy threshold this is rare after the first blocks. O may
        // be touched only after the previous block's P V has finished (P itself no longer waits for it: it lives
        // in this block's own score buffer)
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
          if (!__all_sync(0xffffffffu, mbar_wait(o_done, (i - 1) & 1, abort_flag))) {
            *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_EMPTY); ok = false; break;
          }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t r[32];
            tmem_ld32(tmem_O + lane_off + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * alpha);
            tmem_st32(tmem_O + lane_off + c, r);
          }
          tmem_st_wait();
        }
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_ready[i & 1]);
    }
    // final: O / l -> out
    if (ok && n_blk > 1) {
      // a parity wait may be at most one phase behind the barrier: this thread may not have looked at o_done for
      // many blocks (it waits only when it rescales), so it first catches up with the block before the last (whose
      // predecessor is known to be complete: it ran before the last block's scores)
      if (!__all_sync(0xffffffffu, mbar_wait(o_done, (n_blk - 2) & 1, abort_flag))) {
        *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_FULL); ok = false;
      }
    }
    if (ok && n_blk > 0) {
      if (!__all_sync(0xffffffffu, mbar_wait(o_done, (n_blk - 1) & 1, abort_flag))) {
        *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_FULL); ok = false;
      }
    }
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = a.out + (long(q0 + tile_row0 + row) * a.Hq + head) * D;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t r[32];
        if (n_blk > 0) {
          tmem_ld32(tmem_O + lane_off + c, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0;
        }
        if (row_ok) {
          uint4* dst = reinterpret_cast<uint4*>(orow + c);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]) * inv, __uint_as_float(r[8 * v + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]) * inv, __uint_as_float(r[8 * v + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]) * inv, __uint_as_float(r[8 * v + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]) * inv, __uint_as_float(r[8 * v + 7]) * inv);
            dst[v] = o;
          }
        }
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
thread_local char g_attn_err[256];

template <int D, int BKV>
int launch_prefill(const CUtensorMap* tq, const CUtensorMap* tk, const CUtensorMap* tv, const PrefillArgs& a,
                   dim3 grid, cudaStream_t s) {
  using Cfg = PrefillCfg<D, BKV>;
  auto kfn = prefill_attn_kernel<D, BKV>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess) {
      snprintf(g_attn_err, sizeof(g_attn_err), "prefill attention: cannot set %d bytes of shared memory", Cfg::SMEM);
      return 1;
    }
    attr = true;
  }
  kfn<<<grid, 160, Cfg::SMEM, s>>>(*tq, *tk, *tv, a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(g_attn_err, sizeof(g_attn_err), "prefill attention launch: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}
}  // namespace

const char* prefill_attn_last_error() { return g_attn_err; }

int prefill_attn_launch(const void* q, long T, const void* k_cache, const void* v_cache, long n_cells,
                        long cell_stride, const int* cu_q, const int* ctx_lens, const int* block_table,
                        int table_width, int page, int n_seqs, int max_q_len, int Hq, int Hkv, int D, float scale,
                        int window, int causal, void* out, int* status, cudaStream_t s) {
  if (n_seqs <= 0 || max_q_len <= 0) return 0;
  const int BKV = D >= 128 ? 64 : 128;
  if (page <= 0 || BKV % page != 0 || page % 8 != 0) {
    snprintf(g_attn_err, sizeof(g_attn_err), "prefill attention: page size %d must be a multiple of 8 dividing %d",
             page, BKV);
    return 1;
  }
  if (D != 64 && D != 128 && D != 256) {
    snprintf(g_attn_err, sizeof(g_attn_err), "prefill attention: head dim %d not supported", D);
    return 1;
  }
  // q viewed as [T, Hq, D]; caches as [cells, Hkv, D] with cell pitch cell_stride elements
  const CUtensorMap* tq = tmap_3d(q, uint64_t(D), uint64_t(Hq), uint64_t(T), uint64_t(D) * 2,
                                  uint64_t(Hq) * D * 2, 64, 1, 128, TM_BF16, true);
  const CUtensorMap* tk = tmap_3d(k_cache, uint64_t(D), uint64_t(Hkv), uint64_t(n_cells), uint64_t(D) * 2,
                                  uint64_t(cell_stride) * 2, 64, 1, uint32_t(page), TM_BF16, true);
  const CUtensorMap* tv = tmap_3d(v_cache, uint64_t(D), uint64_t(Hkv), uint64_t(n_cells), uint64_t(D) * 2,
                                  uint64_t(cell_stride) * 2, 64, 1, uint32_t(page), TM_BF16, true);
  if (!tq || !tk || !tv) {
    snprintf(g_attn_err, sizeof(g_attn_err), "prefill attention: %s", tmap_last_error());
    return 1;
  }
  PrefillArgs a{};
  a.cu_q = cu_q; a.ctx_lens = ctx_lens; a.block_table = block_table; a.table_width = table_width; a.page = page;
  a.Hq = Hq; a.Hkv = Hkv; a.scale_log2 = scale * 1.4426950408889634f; a.window = window; a.causal = causal;
  a.out = static_cast<__nv_bfloat16*>(out); a.status = status;
  dim3 grid((max_q_len + 127) / 128, Hq, n_seqs);
  if (D == 64) return launch_prefill<64, 128>(tq, tk, tv, a, grid, s);
  if (D == 128) return launch_prefill<128, 64>(tq, tk, tv, a, grid, s);
  return launch_prefill<256, 64>(tq, tk, tv, a, grid, s);
}

}  // namespace lb
