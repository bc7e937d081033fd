// Multi-head latent attention (MLA) over the paged latent cache, absorbed form, on tcgen05 for sm_100a.
//
// A cache row is [c_kv (512) | k_pe (64)] in bf16: every head of a token reads the SAME row, as key (all 576
// columns) and as value (the first 512). Queries arrive already absorbed into the latent space,
// q_abs = [q_nope W_uk | rope(q_pe)] (576 per head), and the kernel returns o_lat = softmax(q_abs . row) . c_kv
// (512 per head); the caller applies W_uv and the output projection.
//
// One CTA = 64 query rows (G heads x 64/G consecutive tokens of one sequence) over one split of the keys:
//   warp 5 (one lane)  TMA producer: Q tile once, then 64-key latent tiles through the block table into a two-stage
//                      ring (nine 64-column halves per tile, 128-byte swizzle). ONE tile in shared memory serves
//                      both MMAs: K-major B operand of S = Q K^T and MN-major B operand of O += P V.
//   warp 4 (one lane)  MMA issue with M = 64: S (64 x 64, K = 576, 36 instructions) goes to TMEM lanes 16..31 of
//                      each subpartition, O (64 x 512, two N = 256 halves) to lanes 0..15 of ALL 512 columns - the
//                      M = 64 accumulator layout uses half of the lanes, so S and O interleave in the same columns
//                      and the whole value width fits one CTA.
//   warps 0..3         softmax: lanes 16..31 of warp w own S rows 16w..16w+15 (one row per thread: mask, online
//                      softmax in base 2, P written to shared memory as the swizzled K-major A operand), lanes
//                      0..15 own the matching O rows (lazy rescale, final normalisation and store).
// S of tile j+1 is issued as soon as the softmax has read S of tile j, so it runs under the exponentials; O is
// rescaled only when a row maximum grew by more than 2^8, and only while no MMA is in flight.
// Several splits write (max, sum, unnormalised O) partials that attn_combine merges.
// Every wait is bounded; a wait that runs out sets the status word and the CTA unwinds through the common exit.
//
// Counterparts in the reference: the MLA paths of src/cuda/sm80/paged_attn.cuh and src/model/archs/deepseek.rs
// (latent cache rows, absorbed decode).
#include "common.cuh"
#include "kernels.h"
#include "tmap.cuh"

namespace lb {

namespace {

constexpr int MLA_L = 512;                 // latent (value) width
constexpr int MLA_R = 64;                  // rope width
constexpr int MLA_DK = MLA_L + MLA_R;      // 576
constexpr int MLA_HALVES = MLA_DK / 64;    // 9
constexpr int MLA_BKV = 64;
constexpr int MLA_ROWS = 64;
constexpr int MLA_Q_BYTES = MLA_HALVES * MLA_ROWS * 128;    // 73,728
constexpr int MLA_KV_BYTES = MLA_HALVES * MLA_BKV * 128;    // 73,728
constexpr int MLA_P_BYTES = MLA_ROWS * 128;                 // 8,192
constexpr int MLA_SMEM = MLA_Q_BYTES + 2 * MLA_KV_BYTES + MLA_P_BYTES + 256 + 1024;
constexpr float MLA_RESCALE_LOG2 = 8.f;

__device__ __forceinline__ void mla_tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
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
__device__ __forceinline__ void mla_tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

struct MlaArgs {
  const int* cu_q;         // [n_seqs + 1]
  const int* ctx_lens;     // [n_seqs] keys visible after this step
  const int* block_table;  // [n_seqs, table_width]
  int table_width, page;
  int nh, G, TQ;           // heads, heads per tile, tokens per tile (G * TQ == 64)
  int head_blocks, n_splits;
  float scale_log2;
  __nv_bfloat16* out;      // [T, nh, 512] (n_splits == 1)
  float* o_part;           // [T * nh, n_splits, 512]
  float* ml_part;          // [T * nh, n_splits, 2] (max in natural-log units, sum)
  int* status;
};

__global__ void __launch_bounds__(192, 1)
mla_attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmC, const MlaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* kv_s = q_s + MLA_Q_BYTES;                 // [2] latent tiles
  uint8_t* p_s = kv_s + 2 * MLA_KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + MLA_P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;    // [2]
  uint64_t* kv_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;     // [2] S buffers
  uint64_t* s_free = bars + 7;     // [2]
  uint64_t* p_ready = bars + 9;
  uint64_t* o_done = bars + 10;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int seq = blockIdx.y;
  int w = blockIdx.x;
  const int split = w % a.n_splits; w /= a.n_splits;
  const int hb = w % a.head_blocks;
  const int qt = w / a.head_blocks;
  const int q0 = a.cu_q[seq];
  const int q_len = a.cu_q[seq + 1] - q0;
  const int tok0 = qt * a.TQ;                       // first token of this tile within the sequence's step
  if (tok0 >= q_len) return;                        // uniform per CTA, before any barrier or TMEM use
  const int ctx = a.ctx_lens[seq];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&s_free[i], 128); }
    mbar_init(p_ready, 128);
    mbar_init(o_done, 1);
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
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_O = tmem_base;                      // lanes 0..15 of each subpartition, 512 columns
  const uint32_t tmem_S = tmem_base + (16u << 16);        // lanes 16..31, columns 0..127: two S buffers

  // keys visible to the tile: up to the position of its last valid token
  const int toks_here = min(a.TQ, q_len - tok0);
  const int pos0 = ctx - q_len + tok0;                    // absolute position of the tile's first token
  const int kv_hi = min(ctx, pos0 + toks_here);           // exclusive
  const int n_blk_all = (kv_hi + MLA_BKV - 1) / MLA_BKV;
  const int per = (n_blk_all + a.n_splits - 1) / a.n_splits;
  const int blk_lo = split * per;
  const int n_blk = max(0, min(n_blk_all, blk_lo + per) - blk_lo);
  const int* bt = a.block_table + long(seq) * a.table_width;
  const int pages_per_blk = MLA_BKV / a.page;

  if (warp == 5) {
    if (lane == 0 && n_blk > 0) {
      // ---------------------------------------------------------------- TMA producer
      mbar_expect_tx(q_full, MLA_Q_BYTES);
#pragma unroll
      for (int h = 0; h < MLA_HALVES; ++h)
        tma_load_3d(q_s + h * (MLA_ROWS * 128), &tmQ, q_full, h * 64, hb * a.G, q0 + tok0);
      for (int j = 0; j < n_blk; ++j) {
        const int st = j & 1;
        if (j >= 2 && !mbar_wait(&kv_empty[st], ((j >> 1) - 1) & 1, abort_flag)) {
          *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_EMPTY); break;
        }
        uint8_t* dst = kv_s + st * MLA_KV_BYTES;
        mbar_expect_tx(&kv_full[st], MLA_KV_BYTES);
        const int key0 = (blk_lo + j) * MLA_BKV;
        for (int p = 0; p < pages_per_blk; ++p) {
          const int key = key0 + p * a.page;
          // pages past the end of the sequence read a valid page: masked later
          const int pg = (key < ctx) ? bt[key / a.page] : bt[0];
          const int cell = pg * a.page;
#pragma unroll
          for (int h = 0; h < MLA_HALVES; ++h)
            tma_load_2d(dst + h * (MLA_BKV * 128) + p * a.page * 128, &tmC, &kv_full[st], h * 64, cell);
        }
      }
    }
  } else if (warp == 4) {
    if (lane == 0 && n_blk > 0) {
      // ---------------------------------------------------------------- MMA issue
      constexpr uint32_t idesc_s = umma_idesc(64, MLA_BKV, 1, 1, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc(64, 256, 1, 1, 0, 1);   // B (= latent tile as V) is MN-major
      const uint64_t dq0 = umma_desc_k_sw128(smem_u32(q_s));
      const uint64_t dp0 = umma_desc_k_sw128(smem_u32(p_s));
      auto issue_s = [&](int j) {
        // descriptors differ only in the start address (units of 16 bytes, low bits): base + constant
        const uint64_t dk0 = umma_desc_k_sw128(smem_u32(kv_s + (j & 1) * MLA_KV_BYTES));
#pragma unroll
        for (int h = 0; h < MLA_HALVES; ++h) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t off = uint64_t((h * (MLA_ROWS * 128) + k * 32) >> 4);
            umma_f16(tmem_S + (j & 1) * MLA_BKV, dq0 + off, dk0 + off, idesc_s, (h | k) ? 1u : 0u);
          }
        }
        umma_commit(&s_full[j & 1]);
      };
      auto issue_pv = [&](int j) {
        const uint64_t dv0 = umma_desc_mn_sw128(smem_u32(kv_s + (j & 1) * MLA_KV_BYTES), MLA_BKV * 128, 1024);
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
          for (int k = 0; k < MLA_BKV / 16; ++k) {
            // A = P (K-major, 16 keys = 32 B per step); B = 256 latent columns (4 halves) of 16 key rows
            const uint64_t db = dv0 + uint64_t((n * 4 * (MLA_BKV * 128) + k * 16 * 128) >> 4);
            umma_f16(tmem_O + n * 256, dp0 + uint64_t((k * 32) >> 4), db, idesc_o, (j | k) ? 1u : 0u);
          }
        }
        umma_commit(&kv_empty[j & 1]);
        umma_commit(o_done);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag) && mbar_wait(&kv_full[0], 0, abort_flag);
      if (!ok) { *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_FULL); }
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; ok && j < n_blk; ++j) {
        // Two things are owed in this round, in whichever order their inputs arrive: S of tile j+1 (its latent
        // tile has landed and the softmax of tile j-1 has released that S buffer) and PV of tile j (P is ready).
        // Neither waits behind the other: the softmax of tile j may itself wait for S of tile j+1 before a rescale.
        bool s_owed = j + 1 < n_blk, pv_owed = true;
        uint64_t t0 = 0;                     // the clock (a slow read) only once the round has lasted a while
        uint32_t spins = 0;
        while (s_owed || pv_owed) {
          if (s_owed && mbar_test_wait(&kv_full[(j + 1) & 1], ((j + 1) >> 1) & 1) &&
              (j < 1 || mbar_test_wait(&s_free[(j + 1) & 1], (((j + 1) >> 1) - 1) & 1))) {
            tc_fence_after();
            issue_s(j + 1);
            s_owed = false;
          }
          if (pv_owed && mbar_test_wait(p_ready, j & 1)) {
            tc_fence_after();
            issue_pv(j);
            pv_owed = false;
          }
          if ((++spins & 0x3ff) == 0) {
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            if (*abort_flag || now - t0 > LB_WAIT_NS) {
              *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_FLAG); ok = false; break;
            }
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warps
    const bool s_lane = lane >= 16;                         // lanes 16..31: S rows; lanes 0..15: O rows
    const int row = warp * 16 + (lane & 15);                // tile row of this thread (S or O)
    const int tq = row / a.G;                               // token within the tile
    const int head = hb * a.G + row % a.G;
    const bool row_ok = tq < toks_here;
    const int hi = row_ok ? min(ctx, pos0 + tq + 1) : 0;    // exclusive key bound (causal)
    const uint32_t lane_off = uint32_t(warp * 32) << 16;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blk; ++j) {
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[j & 1], (j >> 1) & 1, abort_flag))) {
        *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_FULL); ok = false; break;
      }
      tc_fence_after();
      const int key0 = (blk_lo + j) * MLA_BKV;
      const uint32_t s_col = uint32_t(j & 1) * MLA_BKV;
      // S of row i sits in lane 16 + i: that lane keeps columns 32..63 and hands columns 0..31 to lane i, so both
      // halves of the warp share the exponentials of a row
      uint32_t v[32];
      {
        uint32_t r[MLA_BKV];
        tmem_ld32(tmem_base + lane_off + s_col, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        tmem_ld32(tmem_base + lane_off + s_col + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const uint32_t got = __shfl_down_sync(0xffffffffu, r[c], 16);
          v[c] = s_lane ? r[32 + c] : got;
        }
      }
      // the row's probabilities are computed into registers first: nothing here depends on the previous PV
      const int kc = key0 + (s_lane ? 32 : 0);              // first key of this lane's 32 columns
      const bool full = key0 + MLA_BKV <= hi;               // every key of the tile is visible to this row
      float mx = -INFINITY;
      if (full) {
#pragma unroll
        for (int c = 0; c < 32; ++c) mx = fmaxf(mx, __uint_as_float(v[c]));
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c)
          if (kc + c < hi) mx = fmaxf(mx, __uint_as_float(v[c]));
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      float alpha = 1.f;
      const float m_blk = mx * a.scale_log2;
      if (m_blk > m + MLA_RESCALE_LOG2 || (m == -INFINITY && m_blk != -INFINITY)) {
        alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_blk);
        m = m_blk;
      }
      const float neg_m = (m == -INFINITY) ? 0.f : -m;
      float sum = 0.f;
      uint32_t packed[16];
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        float p0 = exp2f(fmaf(__uint_as_float(v[c]), a.scale_log2, neg_m));
        float p1 = exp2f(fmaf(__uint_as_float(v[c + 1]), a.scale_log2, neg_m));
        if (!full) {
          if (kc + c >= hi) p0 = 0.f;
          if (kc + c + 1 >= hi) p1 = 0.f;
        }
        // sum what the tensor core will see (bf16-rounded): numerator and denominator stay consistent
        const __nv_bfloat162 bb = __floats2bfloat162_rn(p0, p1);
        const float2 ff = __bfloat1622float2(bb);
        sum += ff.x + ff.y;
        packed[c / 2] = *reinterpret_cast<const uint32_t*>(&bb);
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 16);
      l = l * alpha + sum;                                  // (m, l) are kept alike in both lanes of a row
      // lanes 0..15 hold the O rows; lanes 16..31 rewrite S / unused cells unchanged
      const float f = s_lane ? 1.f : alpha;
      bool waited = false;
      if (j >= 1 && __any_sync(0xffffffffu, f != 1.f)) {
        // O is rescaled only while no MMA is in flight: PV of tile j-1 has finished, S of tile j+1 (the only S that
        // can be on its way) has completed, S of tile j+2 waits for this tile's s_free and PV of tile j for p_ready.
        // Lanes 16..31 rewrite what they read (columns 0..127 hold the two S buffers, the rest is unused).
        bool done = mbar_wait(o_done, (j - 1) & 1, abort_flag);
        if (done && j + 1 < n_blk) done = mbar_wait(&s_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, done)) {
          *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_EMPTY); ok = false; break;
        }
        tc_fence_after();
        waited = true;
#pragma unroll 1
        for (int c = 0; c < MLA_L; c += 32) {
          uint32_t o[32];
          tmem_ld32(tmem_base + lane_off + c, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
          mla_tmem_st32(tmem_base + lane_off + c, o);
        }
        mla_tmem_st_wait();
      }
      tc_fence_before();
      mbar_arrive(&s_free[j & 1]);
      // P is overwritten only after the previous PV has read it
      if (j >= 1 && !waited) {
        if (!__all_sync(0xffffffffu, mbar_wait(o_done, (j - 1) & 1, abort_flag))) {
          *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_EMPTY); ok = false; break;
        }
        tc_fence_after();
      }
      {
        uint8_t* prow = p_s + row * 128;
        const int ch0 = s_lane ? 4 : 0;                     // 16-byte chunks of this lane's 32 columns
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int chunk = (ch0 + ch) ^ (row & 7);
          *reinterpret_cast<uint4*>(prow + chunk * 16) =
              make_uint4(packed[4 * ch], packed[4 * ch + 1], packed[4 * ch + 2], packed[4 * ch + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
    }
    if (ok && n_blk > 0) {
      if (!__all_sync(0xffffffffu, mbar_wait(o_done, (n_blk - 1) & 1, abort_flag))) {
        *abort_flag = 1; atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_FULL); ok = false;
      }
    }
    if (ok) {
      tc_fence_after();
      const float m_o = m, l_o = l;
      const long grow = long(q0 + tok0 + tq) * a.nh + head;         // global (token, head) row
      const bool write = !s_lane && row_ok;
      if (a.n_splits == 1) {
        const float inv = l_o > 0.f ? 1.f / l_o : 0.f;
        __nv_bfloat16* orow = a.out + grow * MLA_L;
#pragma unroll 1
        for (int c = 0; c < MLA_L; c += 32) {
          uint32_t o[32];
          if (n_blk > 0) {
            tmem_ld32(tmem_base + lane_off + c, o);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0;
          }
          if (write) {
            uint4* dst = reinterpret_cast<uint4*>(orow + c);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 u;
              u.x = pack_bf16x2(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
              u.y = pack_bf16x2(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
              u.z = pack_bf16x2(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
              u.w = pack_bf16x2(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
              dst[v] = u;
            }
          }
        }
      } else {
        float* orow = a.o_part + (grow * a.n_splits + split) * MLA_L;
        if (write) {
          float* ml = a.ml_part + (grow * a.n_splits + split) * 2;
          ml[0] = (n_blk > 0 && m_o != -INFINITY) ? m_o * 0.6931471805599453f : -INFINITY;
          ml[1] = n_blk > 0 ? l_o : 0.f;
        }
#pragma unroll 1
        for (int c = 0; c < MLA_L; c += 32) {
          uint32_t o[32];
          if (n_blk > 0) {
            tmem_ld32(tmem_base + lane_off + c, o);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0;
          }
          if (write) {
            float4* dst = reinterpret_cast<float4*>(orow + c);
#pragma unroll
            for (int v = 0; v < 8; ++v)
              dst[v] = make_float4(__uint_as_float(o[4 * v]), __uint_as_float(o[4 * v + 1]),
                                   __uint_as_float(o[4 * v + 2]), __uint_as_float(o[4 * v + 3]));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// One block per token: cache row = [rmsnorm(c_kv) * w | rope(k_pe)] written at the token's cell (slot < 0: padding
// row, nothing is written), and rope(q_pe) of every head written into columns 512..575 of q_abs.
// Rotate-half pairing (i, i + 32); cos_sin rows are [cos(32) | sin(32)].
__global__ void __launch_bounds__(128)
mla_prep_kernel(const __nv_bfloat16* __restrict__ kva, long ld_kva, const float* __restrict__ norm_w, float eps,
                float w_offset, const __nv_bfloat16* __restrict__ q, long ld_q_tok, int q_head_stride, int q_pe_off,
                int nh, const float* __restrict__ cos_sin, const int* __restrict__ positions,
                const long* __restrict__ slots, __nv_bfloat16* __restrict__ cache, long cell_stride,
                __nv_bfloat16* __restrict__ q_abs) {
  __shared__ float red[4];
  const int t = blockIdx.x, tid = threadIdx.x;
  const __nv_bfloat16* row = kva + long(t) * ld_kva;
  const float* cs = cos_sin + long(positions[t]) * MLA_R;
  float v[4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[i] = __bfloat162float(row[tid * 4 + i]);
    ss += v[i] * v[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  const float inv = rsqrtf((red[0] + red[1] + red[2] + red[3]) / float(MLA_L) + eps);
  const long slot = slots[t];
  if (slot >= 0) {
    __nv_bfloat16* dst = cache + slot * cell_stride;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      dst[tid * 4 + i] = __float2bfloat16(v[i] * inv * (norm_w[tid * 4 + i] + w_offset));
    if (tid < 32) {
      const float a = __bfloat162float(row[MLA_L + tid]), b = __bfloat162float(row[MLA_L + 32 + tid]);
      const float c = cs[tid], sn = cs[32 + tid];
      dst[MLA_L + tid] = __float2bfloat16(a * c - b * sn);
      dst[MLA_L + 32 + tid] = __float2bfloat16(b * c + a * sn);
    }
  }
  for (int idx = tid; idx < nh * 32; idx += 128) {
    const int h = idx >> 5, i = idx & 31;
    const __nv_bfloat16* qp = q + long(t) * ld_q_tok + long(h) * q_head_stride + q_pe_off;
    const float a = __bfloat162float(qp[i]), b = __bfloat162float(qp[32 + i]);
    const float c = cs[i], sn = cs[32 + i];
    __nv_bfloat16* qo = q_abs + (long(t) * nh + h) * MLA_DK + MLA_L;
    qo[i] = __float2bfloat16(a * c - b * sn);
    qo[32 + i] = __float2bfloat16(b * c + a * sn);
  }
}

thread_local char g_mla_err[256];

}  // namespace

int mla_prep_launch(const void* kva, long ld_kva, const float* norm_w, float eps, float w_offset, const void* q,
                    long ld_q_tok, int q_head_stride, int q_pe_off, int nh, const float* cos_sin,
                    const int* positions, const long* slots, void* cache, long cell_stride, void* q_abs, int T,
                    cudaStream_t s) {
  if (T <= 0) return 0;
  mla_prep_kernel<<<T, 128, 0, s>>>(static_cast<const __nv_bfloat16*>(kva), ld_kva, norm_w, eps, w_offset,
                                    static_cast<const __nv_bfloat16*>(q), ld_q_tok, q_head_stride, q_pe_off, nh,
                                    cos_sin, positions, slots, static_cast<__nv_bfloat16*>(cache), cell_stride,
                                    static_cast<__nv_bfloat16*>(q_abs));
  return cudaGetLastError() != cudaSuccess ? 1 : 0;
}

const char* mla_attn_last_error() { return g_mla_err; }

// q_abs [T, nh, 576] bf16; cache rows [n_cells, 576] bf16 with pitch cell_stride elements; out [T, nh, 512] bf16.
// o_part / ml_part: workspaces of T * nh * n_splits * 512 and T * nh * n_splits * 2 floats (n_splits > 1).
int mla_attn_launch(const void* q_abs, long T, const void* cache, long n_cells, long cell_stride, const int* cu_q,
                    const int* ctx_lens, const int* block_table, int table_width, int page, int n_seqs,
                    int max_q_len, int nh, float scale, int n_splits, float* o_part, float* ml_part, void* out,
                    int* status, cudaStream_t s) {
  if (n_seqs <= 0 || max_q_len <= 0 || T <= 0) return 0;
  if (page <= 0 || MLA_BKV % page != 0 || page % 8 != 0) {
    snprintf(g_mla_err, sizeof(g_mla_err), "mla attention: page size %d must be a multiple of 8 dividing %d", page,
             MLA_BKV);
    return 1;
  }
  int G = nh >= 64 ? 64 : nh;
  if (nh <= 0 || (nh >= 64 && nh % 64 != 0) || (nh < 64 && (64 % nh) != 0)) {
    snprintf(g_mla_err, sizeof(g_mla_err), "mla attention: %d heads (need a divisor or a multiple of 64)", nh);
    return 1;
  }
  if (n_splits < 1) n_splits = 1;
  if (n_splits > 1 && (!o_part || !ml_part)) {
    snprintf(g_mla_err, sizeof(g_mla_err), "mla attention: split keys need the partial workspaces");
    return 1;
  }
  if (cell_stride % 8 != 0) {
    snprintf(g_mla_err, sizeof(g_mla_err), "mla attention: cache row pitch %ld must be a multiple of 8", cell_stride);
    return 1;
  }
  const int TQ = 64 / G;
  const CUtensorMap* tq = tmap_3d(q_abs, uint64_t(MLA_DK), uint64_t(nh), uint64_t(T), uint64_t(MLA_DK) * 2,
                                  uint64_t(nh) * MLA_DK * 2, 64, uint32_t(G), uint32_t(TQ), TM_BF16, true);
  const CUtensorMap* tc = tmap_2d(cache, uint64_t(n_cells), uint64_t(MLA_DK), uint64_t(cell_stride) * 2,
                                  uint32_t(page), 64, TM_BF16, true);
  if (!tq || !tc) {
    snprintf(g_mla_err, sizeof(g_mla_err), "mla attention: %s", tmap_last_error());
    return 1;
  }
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(mla_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MLA_SMEM) != cudaSuccess) {
      snprintf(g_mla_err, sizeof(g_mla_err), "mla attention: cannot set %d bytes of shared memory", MLA_SMEM);
      return 1;
    }
    attr = true;
  }
  MlaArgs a{};
  a.cu_q = cu_q; a.ctx_lens = ctx_lens; a.block_table = block_table; a.table_width = table_width; a.page = page;
  a.nh = nh; a.G = G; a.TQ = TQ; a.head_blocks = nh / G; a.n_splits = n_splits;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.out = static_cast<__nv_bfloat16*>(out); a.o_part = o_part; a.ml_part = ml_part; a.status = status;
  const int q_tiles = (max_q_len + TQ - 1) / TQ;
  dim3 grid(unsigned(q_tiles) * a.head_blocks * n_splits, unsigned(n_seqs));
  mla_attn_kernel<<<grid, 192, MLA_SMEM, s>>>(*tq, *tc, a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(g_mla_err, sizeof(g_mla_err), "mla attention launch: %s", cudaGetErrorString(e));
    return 1;
  }
  if (n_splits > 1) return attn_combine_launch(o_part, ml_part, n_splits, int(T) * nh, MLA_L, out, s);
  return 0;
}

}  // namespace lb
