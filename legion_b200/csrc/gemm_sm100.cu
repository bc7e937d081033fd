// Weights-as-M tcgen05 GEMM for sm_100a ("wgemm").
//
//   out[token, feature] = sum_k W[group*rows_per_group + feature, k] * X[token, k]
//
// The WEIGHT rows are the UMMA M dimension (128 per tile, one TMEM lane each) and the TOKENS are the
// UMMA N dimension (BN = 32..256 accumulator columns). One orientation serves every linear layer of
// the engine: a decode step with 1..64 tokens streams each weight tile exactly once at full TMA depth
// (small BN leaves room for 10+ stages in flight per SM), a prefill chunk uses BN = 256, and the
// routed-expert GEMM is the same kernel walking a device-built list of (expert, token range) tiles.
//
// Roles per CTA (192 threads, persistent over work items):
//   warp 0      TMA producer: weight tile(s) + token tile per 64-wide k block, 128-byte swizzle
//   warp 1      tcgen05.mma issuer (one elected thread), accumulators double-buffered in TMEM
//   warps 2..5  epilogue: tcgen05.ld -> (SwiGLU | row scale | residual) -> global stores; each thread
//               owns one feature row, so for a given token the 32 lanes of a warp write 64 contiguous
//               bytes of the token-major output.
// DUAL mode loads two weight tiles (gate and up rows of the same features) into two accumulators
// and writes silu(gate) * up. Split-K writes fp32 partials to a workspace; the last CTA to arrive at
// a tile sums the partials in split order (deterministic) and runs the epilogue.
//
// Counterpart in the reference: cuBLAS GEMMs reached through ggml, src/cuda/dense_mv.cu (skinny
// BF16), src/cuda/moe_gemm.cu (routed experts, >= 64 tokens), src/cuda/expert_mv/ (decode experts).
#include <cuda_fp16.h>

#include "comm_dev.cuh"
#include "common.cuh"
#include "gemm_sm100.h"
#include "nvfp4_dev.cuh"
#include "tmap.cuh"

namespace lb {

static constexpr int BM = 128;        // weight rows per tile
static constexpr int BK = 64;         // bf16 elements per k block = one 128-byte swizzle row
static constexpr int UMMA_K = 16;
static constexpr int W_TILE_BYTES = BM * BK * 2;  // 16 KiB
static constexpr int SMEM_BUDGET = 200 * 1024;

static constexpr int W_RAW_BYTES = BM * BK / 2;   // NVFP4: 128 rows x 32 bytes of packed e2m1 codes per k block
static constexpr int W_SC_BYTES = BM * 16;        //        128 rows x 16 e4m3 block scales (4 k blocks of 64)

template <int BN, bool DUAL, bool WFP4 = false, bool WFP8 = false>
struct WgemmCfg {
  static constexpr int NW = DUAL ? 2 : 1;
  static constexpr int X_TILE_BYTES = BN * BK * 2;
  static constexpr int X_OFF = W_TILE_BYTES * NW;                 // operand tiles first (1024-byte aligned)
  static constexpr int RAW_OFF = X_OFF + X_TILE_BYTES;            // NVFP4 only: packed codes, then block scales
  static constexpr int SC_OFF = RAW_OFF + W_RAW_BYTES * NW;
  static constexpr int STAGE_BYTES = WFP4 ? SC_OFF + W_SC_BYTES * NW : RAW_OFF;
  static constexpr int THREADS = WFP4 ? 448 : 192;                // NVFP4 adds 8 de-quantisation warps
  static constexpr int LUT_BYTES = WFP4 ? 512 : 0;                // e4m3 byte -> f16 table
  static constexpr int STAGES_RAW = SMEM_BUDGET / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 12 ? 12 : STAGES_RAW;
  static constexpr int ACC_COLS = BN * (DUAL ? 2 : 1);
  // bf16 / NVFP4: two accumulators (one drains while the next tile runs). FP8: a ring of four PARTIAL accumulators,
  // one per 128-wide k block, which the epilogue warps scale and add up in registers
  static constexpr int NACC = WFP8 ? 4 : 2;
  static constexpr int TMEM_COLS = NACC * ACC_COLS < 32 ? 32 : NACC * ACC_COLS;
  static constexpr int EPI_BYTES = 32 * BM * 4;  // fp32 staging of 32 token columns
  static constexpr int SMEM_BYTES =
      STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*align slack*/ + 512 /*barriers*/ + LUT_BYTES;
  static_assert(TMEM_COLS <= 512, "accumulators do not fit TMEM");
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0, "TMEM column count must be a power of two");
};

struct WorkItem {
  int group, tok0, out0, ntok, feat0, ks, tile_id;   // tok0: first x row; out0: first output row
};

template <int BN>
__device__ __forceinline__ bool decode_work(const WgemmArgs& a, int w, int n_tok_tiles, WorkItem& it) {
  const int per_tok_tile = a.feat_tiles * a.split_k;
  const int tt = w / per_tok_tile;
  if (tt >= n_tok_tiles) return false;
  const int r = w - tt * per_tok_tile;
  const int ft = r / a.split_k;
  it.ks = r - ft * a.split_k;
  it.feat0 = ft * BM;
  it.tile_id = tt * a.feat_tiles + ft;
  if (a.tile_group) {
    it.group = a.tile_group[tt];
    it.tok0 = a.tile_tok0[tt];
    it.out0 = a.tile_out0 ? a.tile_out0[tt] : it.tok0;
    it.ntok = a.tile_ntok[tt];
  } else {
    it.group = 0;
    it.tok0 = tt * BN;
    it.out0 = it.tok0;
    it.ntok = min(BN, a.n_tok - it.tok0);
  }
  return true;
}

// e4m3 (fn) byte -> f16 bits; every e4m3 value is exact in f16
__device__ __forceinline__ uint32_t e4m3_f16_bits(uint32_t b) {
  const uint32_t e = (b >> 3) & 15u, m = b & 7u;
  float v;
  if (e == 0u) v = float(m) * 0.001953125f;                     // subnormals: m * 2^-9
  else if (e == 15u && m == 7u) v = 0.f;                         // NaN pattern: treated as 0
  else v = __uint_as_float(((e + 120u) << 23) | (m << 20));
  return uint32_t(__half_as_ushort(__float2half_rn(v))) | ((b & 0x80u) << 8);
}
// four bytes of e2m1 code pairs -> four f16x2 words (hardware conversion, exact)
__device__ __forceinline__ void e2m1x8_to_f16x2(uint32_t pk, uint32_t (&o)[4]) {
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\tcvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=r"(o[0]), "=r"(o[1]), "=r"(o[2]), "=r"(o[3]) : "r"(pk));
}
// bf16x2 -> f16x2, clamped to the f16 range
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
  const float lo = fminf(fmaxf(__uint_as_float(v << 16), -65504.f), 65504.f);
  const float hi = fminf(fmaxf(__uint_as_float(v & 0xFFFF0000u), -65504.f), 65504.f);
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <int BN, bool DUAL, bool OUT_F32, bool WFP4, bool WFP8 = false>
__global__ void __launch_bounds__(WFP4 ? 448 : 192, 1)
wgemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
             const __grid_constant__ CUtensorMap tmS, const WgemmArgs a) {
  using Cfg = WgemmCfg<BN, DUAL, WFP4, WFP8>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int NACC = Cfg::NACC;
  constexpr int KBE = WFP8 ? 128 : BK;     // elements per k block: one 128-byte swizzle row of e4m3 or bf16
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* stage = reinterpret_cast<float*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES + Cfg::EPI_BYTES);
  uint64_t* full = bars;                  // [STAGES]
  uint64_t* empty = bars + STAGES;        // [STAGES]
  uint64_t* tfull = bars + 2 * STAGES;    // [NACC]
  uint64_t* tempty = bars + 2 * STAGES + 4;  // [NACC]
  uint64_t* wready = bars + 2 * STAGES + 8;  // [STAGES] NVFP4: operand tile of the stage has been expanded
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 8 + (WFP4 ? STAGES : 0));
  uint16_t* lut_sc = reinterpret_cast<uint16_t*>(smem + STAGES * Cfg::STAGE_BYTES + Cfg::EPI_BYTES + 512);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_flag = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      if (WFP4) mbar_init(&wready[s], 256);
    }
    for (int i = 0; i < NACC; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4);  // one arrive per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if (WFP4 && threadIdx.x >= 192) {      // conversion tables, built by the de-quantisation warps
    const uint32_t b = threadIdx.x - 192;                       // 0..255
    lut_sc[b] = uint16_t(e4m3_f16_bits(b));
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // barriers, TMEM and descriptors are set up: from here on global memory is touched
  griddep_wait();
  griddep_launch();

  // ------------------------------------------------------------------ fused all-gather of the activation rows
  // Flag round with the peers (their shards were written by earlier kernels), then all CTAs of this persistent
  // grid copy the ranks' row blocks over NVLink peer loads into the local operand tensor, meet at a grid-wide
  // arrive, and only then do the TMA loads of X start: all-gather and GEMM are one launch.
  if (a.head.enabled) {
    const WgemmCommHead& hd = a.head;
    const uint32_t seq = *reinterpret_cast<const volatile uint32_t*>(hd.seq_ptr) + 1;
    if (blockIdx.x == 0 && threadIdx.x < hd.peers.world) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(hd.peers.signal[threadIdx.x]) + hd.slot_base + hd.peers.rank, seq);
    }
    if (threadIdx.x == 0) *last_flag = 1;
    __syncthreads();
    if (threadIdx.x < hd.peers.world) {
      const uint32_t* mine =
          reinterpret_cast<const uint32_t*>(hd.peers.signal[hd.peers.rank]) + hd.slot_base + threadIdx.x;
      if (!wait_flag_geq(mine, seq, hd.budget_ns)) {
        *last_flag = 0;
        atomicCAS(hd.status, 0, ST_TIMEOUT_FLAG);
      }
    }
    __syncthreads();
    if (*last_flag) {
      const int nv = hd.K / 8;
      const long total = long(hd.T) * nv;
      for (long i = long(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
        const int row = int(i / nv), v = int(i % nv);
        int owner = row / hd.rows_per_rank;
        if (owner >= hd.peers.world) owner = hd.peers.world - 1;
        const uint4 u = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(hd.peers.buffer[owner]) +
                                                       hd.src_off + long(row) * hd.K * 2)[v];
        reinterpret_cast<uint4*>(hd.x_local + long(row) * hd.K)[v] = u;
      }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      atomicAdd(&hd.ctrs[0], 1u);
      uint64_t t0 = 0;
      uint32_t spins = 0;
      while (*reinterpret_cast<volatile unsigned int*>(&hd.ctrs[0]) < gridDim.x) {     // every CTA has copied
        if ((++spins & 0x3f) == 0) {
          const uint64_t now = globaltimer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > hd.budget_ns) {
            atomicCAS(hd.status, 0, ST_TIMEOUT_FLAG);
            break;
          }
        }
      }
      __threadfence();
      const unsigned int old = atomicAdd(&hd.ctrs[1], 1u);       // last one out resets and publishes the sequence
      if (old == gridDim.x - 1) {
        hd.ctrs[0] = 0;
        hd.ctrs[1] = 0;
        *reinterpret_cast<volatile uint32_t*>(hd.seq_ptr) = seq;
      }
    }
    __syncthreads();
    asm volatile("fence.proxy.async;" ::: "memory");   // generic-proxy stores above -> TMA reads below
  }

  const int n_tok_tiles = a.tile_group ? min(*a.n_tiles_dev, a.n_tok_tiles_max) : (a.n_tok + BN - 1) / BN;
  const int num_kb = (a.K + KBE - 1) / KBE;
  const int kb_per_split = (num_kb + a.split_k - 1) / a.split_k;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmW);
      tma_prefetch_desc(&tmX);
      int s = 0;
      uint32_t ph = 0;
      int issued = 0;
      bool ok = true;
      WorkItem it;
      for (int w = blockIdx.x; ok && decode_work<BN>(a, w, n_tok_tiles, it); w += gridDim.x) {
        const int kb0 = it.ks * kb_per_split;
        const int kb1 = min(num_kb, kb0 + kb_per_split);
        const int wrow = it.group * a.rows_per_group + it.feat0;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) {
            *abort_flag = 1;
            atomicCAS(a.status, 0, ST_TIMEOUT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* st = smem + s * Cfg::STAGE_BYTES;
          if (WFP4) {
            // packed codes of this k block; the block scales come 4 k blocks (16 bytes per row) at a time
            const bool sc = (kb % 4 == 0) || kb == kb0;
            mbar_expect_tx(&full[s], Cfg::X_TILE_BYTES + Cfg::NW * (W_RAW_BYTES + (sc ? W_SC_BYTES : 0)));
            tma_load_2d(st + Cfg::RAW_OFF, &tmW, &full[s], kb * (BK / 2), wrow);
            if (DUAL) tma_load_2d(st + Cfg::RAW_OFF + W_RAW_BYTES, &tmW, &full[s], kb * (BK / 2), wrow + a.dual_offset);
            if (sc) {
              tma_load_2d(st + Cfg::SC_OFF, &tmS, &full[s], (kb / 4) * 16, wrow);
              if (DUAL) tma_load_2d(st + Cfg::SC_OFF + W_SC_BYTES, &tmS, &full[s], (kb / 4) * 16, wrow + a.dual_offset);
            }
          } else {
            mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
            tma_load_2d(st, &tmW, &full[s], kb * KBE, wrow);
            if (DUAL) tma_load_2d(st + W_TILE_BYTES, &tmW, &full[s], kb * KBE, wrow + a.dual_offset);
          }
          tma_load_2d(st + Cfg::X_OFF, &tmX, &full[s], it.group * a.x_group_col + kb * KBE, it.tok0);
          ++issued;
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (!ok) {
        // Unwinding: give copies already in flight a bounded time to land before smem is released.
        const int n = issued < STAGES ? issued : STAGES;
        for (int i = 0; i < n; ++i) {
          int si = s - 1 - i;
          uint32_t p = ph;
          if (si < 0) { si += STAGES; p ^= 1; }
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&full[si], p) && globaltimer_ns() - t0 < 2000000ull) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = (WFP4 || WFP8) ? umma_idesc(BM, BN, 0, 0, 0, 0)   // f16 tiles (de-quantiser) / e4m3
                                                : umma_idesc(BM, BN, 1, 1, 0, 0);
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      WorkItem it;
      for (int w = blockIdx.x; ok && decode_work<BN>(a, w, n_tok_tiles, it); w += gridDim.x) {
        const int kb0 = it.ks * kb_per_split;
        const int kb1 = min(num_kb, kb0 + kb_per_split);
        if (!WFP8) {
          if (!mbar_wait(&tempty[acc], acc_ph ^ 1, abort_flag)) {
            *abort_flag = 1;
            atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_EMPTY);
            break;
          }
          tc_fence_after();
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[s], ph, abort_flag) || (WFP4 && !mbar_wait(&wready[s], ph, abort_flag))) {
            *abort_flag = 1;
            atomicCAS(a.status, 0, ST_TIMEOUT_FULL);
            ok = false;
            break;
          }
          if (WFP8 && !mbar_wait(&tempty[acc], acc_ph ^ 1, abort_flag)) {   // this k block's partial accumulator
            *abort_flag = 1;
            atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_EMPTY);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d0 = tmem_base + acc * Cfg::ACC_COLS;
          const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
          const uint64_t dw = umma_desc_k_sw128(sa);
          const uint64_t dw2 = umma_desc_k_sw128(sa + W_TILE_BYTES);
          const uint64_t dx = umma_desc_k_sw128(sa + Cfg::X_OFF);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // one instruction covers 32 bytes of K: 16 bf16 / f16 or 32 e4m3
            const uint64_t koff = uint64_t(k * UMMA_K * 2 / 16);
            if (WFP8) {
              umma_f8(d0, dw + koff, dx + koff, idesc, k > 0 ? 1u : 0u);
              if (DUAL) umma_f8(d0 + BN, dw2 + koff, dx + koff, idesc, k > 0 ? 1u : 0u);
            } else {
              const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
              umma_f16(d0, dw + koff, dx + koff, idesc, accum);
              if (DUAL) umma_f16(d0 + BN, dw2 + koff, dx + koff, idesc, accum);
            }
          }
          umma_commit(&empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
          if (WFP8) {
            umma_commit(&tfull[acc]);
            if (++acc == NACC) { acc = 0; acc_ph ^= 1; }
          }
        }
        if (!ok) break;
        if (!WFP8) {
          umma_commit(&tfull[acc]);
          if (++acc == NACC) { acc = 0; acc_ph ^= 1; }
        }
      }
    }
  } else if (WFP4 && warp >= 6) {
    // ------------------------------------------------------------------ NVFP4 de-quantisation (warps 6..13)
    // The 256 threads expand every weight tile of a stage (128 rows x 64 codes) into the bf16, 128-byte-swizzled
    // operand tile the MMA reads. A task is one 16-byte chunk (8 codes = 4 packed bytes): lane -> (row, chunk)
    // such that a warp reads 128 contiguous bytes of codes and writes four complete 128-byte rows, so neither
    // side has a shared-memory bank conflict. Codes become f16 pairs with the hardware conversion
    // (cvt.rn.f16x2.e2m1x2) and are multiplied by the block scale as f16x2 (exact: 1 + 3 mantissa bits, range
    // 2^-10 .. 2688); the MMA of this variant runs on f16 operands, so the bf16 activation tile of the stage is
    // converted in place as well (clamped to the f16 range).
    const int d = threadIdx.x - 192;
    const int dw = d >> 5, dl = d & 31;
    const int chunk = dl & 7;
    const int row0 = dw * 4 + (dl >> 3);           // rows row0 + 32 * i, i = 0..3
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    uint32_t scw[Cfg::NW][4][4];                   // [tile][row i][k block within the group of 4]: 4 scale bytes
#pragma unroll
    for (int t = 0; t < Cfg::NW; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) scw[t][i][k] = 0u;
    WorkItem it;
    for (int w = blockIdx.x; decode_work<BN>(a, w, n_tok_tiles, it); w += gridDim.x) {
      const int kb0 = it.ks * kb_per_split;
      const int kb1 = min(num_kb, kb0 + kb_per_split);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (ok && !mbar_wait(&full[s], ph, abort_flag)) {
          *abort_flag = 1;
          atomicCAS(a.status, 0, ST_TIMEOUT_FULL);
          ok = false;      // keep arriving so that nobody is left waiting on wready
        }
        uint8_t* st = smem + s * Cfg::STAGE_BYTES;
        if (ok) {
          const bool new_sc = (kb % 4 == 0) || kb == kb0;
          const int kq = kb & 3;
#pragma unroll
          for (int t = 0; t < Cfg::NW; ++t) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int row = row0 + 32 * i;
              if (new_sc) {
                const uint4 v = *reinterpret_cast<const uint4*>(st + Cfg::SC_OFF + t * W_SC_BYTES + row * 16);
                scw[t][i][0] = v.x; scw[t][i][1] = v.y; scw[t][i][2] = v.z; scw[t][i][3] = v.w;
              }
              const uint32_t sw = kq == 0 ? scw[t][i][0] : (kq == 1 ? scw[t][i][1] : (kq == 2 ? scw[t][i][2] : scw[t][i][3]));
              const uint32_t sb = lut_sc[(sw >> (8 * (chunk >> 1))) & 0xFFu];     // scale of this chunk's 16 block
              const uint32_t sc2 = sb | (sb << 16);
              const uint32_t pk = *reinterpret_cast<const uint32_t*>(st + Cfg::RAW_OFF + t * W_RAW_BYTES + row * 32 + chunk * 4);
              uint32_t o[4];
              e2m1x8_to_f16x2(pk, o);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&o[j]),
                                          *reinterpret_cast<const __half2*>(&sc2));
                o[j] = *reinterpret_cast<const uint32_t*>(&r);
              }
              *reinterpret_cast<uint4*>(st + t * W_TILE_BYTES + row * 128 + ((chunk ^ (row & 7)) * 16)) =
                  make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
          // the activations arrive as bf16: convert the X tile in place (chunk positions are unchanged)
          uint4* xt = reinterpret_cast<uint4*>(st + Cfg::X_OFF);
#pragma unroll
          for (int idx = d; idx < BN * 8; idx += 256) {
            uint4 v = xt[idx];
            v.x = bf16x2_to_f16x2(v.x); v.y = bf16x2_to_f16x2(v.y);
            v.z = bf16x2_to_f16x2(v.z); v.w = bf16x2_to_f16x2(v.w);
            xt[idx] = v;
          }
          fence_proxy_async_smem();
        }
        mbar_arrive(&wready[s]);
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_ph = 0;
    WorkItem it;
    for (int w = blockIdx.x; decode_work<BN>(a, w, n_tok_tiles, it); w += gridDim.x) {
      const int row = q * 32 + lane;               // row within the tile
      const int feat = it.feat0 + row;
      const bool feat_ok = feat < a.n_feat;
      // FP8: the tile's result is built here, in registers: every 128-wide k block arrives as its own partial
      // accumulator and is added with the product of the weight block's scale and the token's group scale
      float accg[WFP8 ? BN : 1], accu[(WFP8 && DUAL) ? BN : 1];
      if constexpr (WFP8) {
#pragma unroll
        for (int j = 0; j < BN; ++j) {
          accg[j] = 0.f;
          if (DUAL) accu[j] = 0.f;
        }
        const int kb0 = it.ks * kb_per_split;
        const int kb1 = min(num_kb, kb0 + kb_per_split);
        const long wblk = long((it.group * a.rows_per_group + it.feat0) >> 7) * num_kb;
        const long wblk2 = long((it.group * a.rows_per_group + it.feat0 + a.dual_offset) >> 7) * num_kb;
        bool failed = false;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(&tfull[acc], acc_ph, abort_flag))) {
            *abort_flag = 1;
            atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_FULL);
            failed = true;
            break;
          }
          tc_fence_after();
          const float sw = a.w_bscale[wblk + kb];
          const float sw2 = DUAL ? a.w_bscale[wblk2 + kb] : 0.f;
          const uint32_t tp = tmem_base + (uint32_t(q * 32) << 16) + acc * Cfg::ACC_COLS;
#pragma unroll
          for (int c = 0; c < BN; c += 32) {
            uint32_t r[32], r2[32];
            tmem_ld32(tp + c, r);
            if (DUAL) tmem_ld32(tp + BN + c, r2);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float xs = (c + j < it.ntok) ? __ldg(&a.x_bscale[long(it.tok0 + c + j) * num_kb + kb]) : 0.f;
              accg[c + j] = fmaf(__uint_as_float(r[j]), sw * xs, accg[c + j]);
              if (DUAL) accu[c + j] = fmaf(__uint_as_float(r2[j]), sw2 * xs, accu[c + j]);
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty[acc]);
          if (++acc == NACC) { acc = 0; acc_ph ^= 1; }
        }
        if (failed) break;
      } else {
        if (!__all_sync(0xffffffffu, mbar_wait(&tfull[acc], acc_ph, abort_flag))) {
          *abort_flag = 1;
          atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_FULL);
          break;
        }
        tc_fence_after();
      }
      const uint32_t t0 = tmem_base + (uint32_t(q * 32) << 16) + acc * Cfg::ACC_COLS;
      // 32 accumulator columns starting at column c: from TMEM, or (FP8) from the registers above
      auto load_cols = [&](int c, uint32_t (&r)[32]) {
        if constexpr (WFP8) {
#pragma unroll
          for (int cc = 0; cc < Cfg::ACC_COLS; cc += 32) {
            if (cc == c) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                float v = 0.f;
                if (cc < BN) v = accg[(cc + j) % BN];
                else if constexpr (DUAL) v = accu[(cc + j) % BN];
                r[j] = __float_as_uint(v);
              }
            }
          }
        } else {
          tmem_ld32(t0 + c, r);
          tmem_ld_wait();
        }
      };

      bool finalize = true;
      if (a.split_k > 1) {
        // fp32 partials: ws[tile][split][col][128 rows]
        float* wsp = a.ws + (size_t(it.tile_id) * a.split_k + it.ks) * (Cfg::ACC_COLS * BM);
#pragma unroll 1
        for (int c = 0; c < Cfg::ACC_COLS; c += 32) {
          uint32_t r[32];
          load_cols(c, r);
#pragma unroll
          for (int j = 0; j < 32; ++j) wsp[(c + j) * BM + row] = __uint_as_float(r[j]);
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
          const int old = atomicAdd(&a.counters[it.tile_id], 1);
          *last_flag = (old == a.split_k - 1) ? 1 : 0;
          if (old == a.split_k - 1) a.counters[it.tile_id] = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        finalize = (*last_flag != 0);
        if (finalize) __threadfence();
      }

      if (finalize) {
        const float* wsb = a.split_k > 1 ? a.ws + size_t(it.tile_id) * a.split_k * (Cfg::ACC_COLS * BM) : nullptr;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          if (c >= it.ntok) break;
          float g[32], u[32];
          if (a.split_k > 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) { g[j] = 0.f; u[j] = 0.f; }
            for (int sp = 0; sp < a.split_k; ++sp) {
              const float* p = wsb + size_t(sp) * (Cfg::ACC_COLS * BM);
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                g[j] += __ldcg(&p[(c + j) * BM + row]);
                if (DUAL) u[j] += __ldcg(&p[(BN + c + j) * BM + row]);
              }
            }
          } else {
            uint32_t r[32];
            load_cols(c, r);
#pragma unroll
            for (int j = 0; j < 32; ++j) g[j] = __uint_as_float(r[j]);
            if (DUAL) {
              load_cols(BN + c, r);
#pragma unroll
              for (int j = 0; j < 32; ++j) u[j] = __uint_as_float(r[j]);
            }
          }
          if (WFP4 && a.w_gscale) {          // per-tensor (per-expert) scale of the NVFP4 encoding
            const float gs0 = a.w_gscale[it.group * Cfg::NW], gs1 = DUAL ? a.w_gscale[it.group * 2 + 1] : 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              g[j] *= gs0;
              if (DUAL) u[j] *= gs1;
            }
          }
          if (!OUT_F32 && a.vec_ok) {
            // Staged write-out: fp32 values go through shared memory so that every token row leaves as
            // 16-byte stores covering 256 contiguous bytes per 16 lanes (8 token rows per pass).
            const int etid = threadIdx.x - 64;  // 0..127 over the four epilogue warps
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float v = g[j];
              if (DUAL) v = (v / (1.f + __expf(-v))) * u[j];
              stage[j * BM + row] = v;
            }
            asm volatile("bar.sync 2, 128;" ::: "memory");
            const int f8 = (etid & 15) * 8;          // first of 8 features handled by this thread
            const int feat8 = it.feat0 + f8;
            if constexpr (WFP8 && DUAL) {
              if (a.q8_out) {
                // Encoded write-out: the 16 lanes that hold one token's 128 features of this tile own exactly one
                // scale group of the next FP8 GEMM: largest magnitude over the half-warp, then 8 e4m3 bytes per lane.
                // Values are rounded to bf16 first, so the bytes are those the activation encoder makes of bf16 rows.
#pragma unroll
                for (int pass = 0; pass < 4; ++pass) {
                  const int j = pass * 8 + (etid >> 4);
                  const int t = c + j;
                  const float4 v0 = *reinterpret_cast<const float4*>(&stage[j * BM + f8]);
                  const float4 v1 = *reinterpret_cast<const float4*>(&stage[j * BM + f8 + 4]);
                  float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                  float amax = 0.f;
#pragma unroll
                  for (int e = 0; e < 8; ++e) {
                    v[e] = __bfloat162float(__float2bfloat16(v[e]));
                    amax = fmaxf(amax, fabsf(v[e]));
                  }
#pragma unroll
                  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                  const float sc = amax > 0.f ? amax / 448.f : 1.f;
                  const float inv = 1.f / sc;
                  if (t < it.ntok) {
                    const long orow = it.out0 + t;
                    uint2 o;
                    o.x = e4m3_enc(v[0] * inv) | (e4m3_enc(v[1] * inv) << 8) | (e4m3_enc(v[2] * inv) << 16) |
                          (e4m3_enc(v[3] * inv) << 24);
                    o.y = e4m3_enc(v[4] * inv) | (e4m3_enc(v[5] * inv) << 8) | (e4m3_enc(v[6] * inv) << 16) |
                          (e4m3_enc(v[7] * inv) << 24);
                    *reinterpret_cast<uint2*>(a.q8_out + orow * a.n_feat + feat8) = o;
                    if ((etid & 15) == 0) a.q8_scale[orow * (a.n_feat >> 7) + (it.feat0 >> 7)] = sc;
                  }
                }
                asm volatile("bar.sync 2, 128;" ::: "memory");
                continue;
              }
            }
#pragma unroll
            for (int pass = 0; pass < 4; ++pass) {
              const int j = pass * 8 + (etid >> 4);
              const int t = c + j;
              if (t < it.ntok && feat8 < a.n_feat) {
                const int xrow = it.out0 + t;
                long orow = xrow;
                if (a.out_rows) orow = a.out_rows[xrow];
                if (orow >= 0) {
                  __nv_bfloat16* obase = reinterpret_cast<__nv_bfloat16*>(a.out);
                  if (a.n_out_peer > 0) {
                    obase = reinterpret_cast<__nv_bfloat16*>(a.out_peer[(orow >> 24) & 7]);
                    orow &= 0xffffff;
                  }
                  const float4 v0 = *reinterpret_cast<const float4*>(&stage[j * BM + f8]);
                  const float4 v1 = *reinterpret_cast<const float4*>(&stage[j * BM + f8 + 4]);
                  float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                  if (a.tok_scale) {
                    const float sc = a.tok_scale[xrow];
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] *= sc;
                  }
                  if (a.residual) {
                    const uint4 rr = *reinterpret_cast<const uint4*>(a.residual + orow * a.ldr + feat8);
                    const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                      const float2 f = __bfloat1622float2(r2[e]);
                      v[2 * e] += f.x;
                      v[2 * e + 1] += f.y;
                    }
                  }
                  uint4 o;
                  o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
                  o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
                  *reinterpret_cast<uint4*>(obase + orow * a.ldo + feat8) = o;
                }
              }
            }
            asm volatile("bar.sync 2, 128;" ::: "memory");
          } else if (feat_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int t = c + j;
              if (t < it.ntok) {
                const int xrow = it.out0 + t;
                float v = g[j];
                if (DUAL) v = (v / (1.f + __expf(-v))) * u[j];
                if (a.tok_scale) v *= a.tok_scale[xrow];
                long orow = xrow;
                if (a.out_rows) orow = a.out_rows[xrow];
                if (orow >= 0) {
                  void* obase = a.out;
                  if (a.n_out_peer > 0) {
                    obase = a.out_peer[(orow >> 24) & 7];
                    orow &= 0xffffff;
                  }
                  if (a.residual) v += __bfloat162float(a.residual[orow * a.ldr + feat]);
                  if (OUT_F32) {
                    reinterpret_cast<float*>(obase)[orow * a.ldo + feat] = v;
                  } else {
                    reinterpret_cast<__nv_bfloat16*>(obase)[orow * a.ldo + feat] = __float2bfloat16(v);
                  }
                }
              }
            }
          }
        }
      }
      if (!WFP8) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
        if (++acc == NACC) { acc = 0; acc_ph ^= 1; }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }

  // ------------------------------------------------------------------ fused reduction over the ranks
  // The output tiles written above are this rank's PARTIAL result inside its symmetric buffer. All CTAs of this
  // (persistent, fully resident) grid count themselves in; the last one raises this rank's flag on every peer;
  // every CTA then waits (bounded) for all ranks' flags and reduces its share of the rows over NVLink peer
  // loads in rank order, adding the residual and applying the next RMSNorm: GEMM and all-reduce are one launch.
  if (a.comm.enabled) {
    const WgemmCommTail& c = a.comm;
    float* red = stage;                         // epilogue staging memory is idle now
    __threadfence_system();                     // this thread's partial stores, system scope
    __syncthreads();
    const uint32_t seq = *reinterpret_cast<const volatile uint32_t*>(c.seq_ptr) + 1;
    if (threadIdx.x == 0) {
      const unsigned int old = atomicAdd(&c.ctrs[0], 1u);
      *last_flag = (old == gridDim.x - 1);
      if (old == gridDim.x - 1) c.ctrs[0] = 0;
    }
    __syncthreads();
    if (*last_flag && threadIdx.x < c.peers.world) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(c.peers.signal[threadIdx.x]) + c.slot_base + c.peers.rank, seq);
    }
    __syncthreads();
    if (threadIdx.x == 0) *last_flag = 1;       // reused as "all peers arrived"
    __syncthreads();
    if (threadIdx.x < c.peers.world) {
      const uint32_t* mine =
          reinterpret_cast<const uint32_t*>(c.peers.signal[c.peers.rank]) + c.slot_base + threadIdx.x;
      if (!wait_flag_geq(mine, seq, c.budget_ns)) {
        *last_flag = 0;
        atomicCAS(c.status, 0, ST_TIMEOUT_FLAG);
      }
    }
    __syncthreads();
    if (*last_flag)
      reduce_rows_rank_order(c.peers, c.buf_off, c.T, c.H, c.residual, c.ldr, c.sum_out, c.lds, c.norm_w, c.eps,
                             c.w_offset, c.norm_out, c.ldn, red);
    // the last CTA to finish publishes the new sequence number (every CTA has read the old one)
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      const unsigned int old = atomicAdd(&c.ctrs[1], 1u);
      if (old == gridDim.x - 1) {
        c.ctrs[1] = 0;
        *reinterpret_cast<volatile uint32_t*>(c.seq_ptr) = seq;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
namespace {

thread_local char g_gemm_err[512];

template <int BN, bool DUAL, bool OUT_F32, bool WFP4 = false, bool WFP8 = false>
int launch(const CUtensorMap* tmW, const CUtensorMap* tmX, const CUtensorMap* tmS, const WgemmArgs& a, int grid,
           cudaStream_t stream) {
  using Cfg = WgemmCfg<BN, DUAL, WFP4, WFP8>;
  auto kfn = wgemm_kernel<BN, DUAL, OUT_F32, WFP4, WFP8>;
  static bool attr_set = false;  // per instantiation
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) {
      snprintf(g_gemm_err, sizeof(g_gemm_err), "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return 1;
    }
    attr_set = true;
  }
  launch_pdl(kfn, dim3(grid), dim3(Cfg::THREADS), Cfg::SMEM_BYTES, stream, *tmW, *tmX, *tmS, a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(g_gemm_err, sizeof(g_gemm_err), "wgemm launch: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

int g_num_sms = 0;

}  // namespace

int wgemm_pick_bn(int n_tok_per_tile_hint, bool dual) {
  int bn = 32;
  while (bn < n_tok_per_tile_hint && bn < (dual ? 128 : 256)) bn *= 2;
  return bn;
}

size_t wgemm_workspace_floats(int bn, bool dual, int n_tok_tiles, int feat_tiles, int split_k) {
  if (split_k <= 1) return 0;
  return size_t(n_tok_tiles) * feat_tiles * split_k * (bn * (dual ? 2 : 1)) * BM;
}

const char* wgemm_last_error() { return g_gemm_err; }

int wgemm_launch(const WgemmHost& h, cudaStream_t stream) {
  if (h.K % 8 != 0) {
    snprintf(g_gemm_err, sizeof(g_gemm_err), "wgemm: K=%d must be a multiple of 8 (16-byte TMA rows)", h.K);
    return 1;
  }
  if ((reinterpret_cast<uintptr_t>(h.w) | reinterpret_cast<uintptr_t>(h.x)) & 15) {
    snprintf(g_gemm_err, sizeof(g_gemm_err), "wgemm: operand base addresses must be 16-byte aligned");
    return 1;
  }
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  const int bn = h.bn;
  const bool fp4 = h.w_scales != nullptr;
  const bool fp8 = h.w_bscale != nullptr;
  if (fp8) {
    // e4m3 operands straight into the f8f6f4 MMA; scales per 128 x 128 weight block and per token and 128 columns
    if (fp4 || !h.x_bscale || h.K % 128 != 0 || h.out_f32 || (bn != 32 && bn != 64) || h.rows_per_group % 128 != 0 ||
        (h.dual && h.dual_offset % 128 != 0) || h.ldw % 16 != 0 || h.ldx % 16 != 0 || h.comm.enabled || h.head.enabled) {
      snprintf(g_gemm_err, sizeof(g_gemm_err),
               "wgemm: FP8 needs K %% 128 == 0, token tiles of 32 or 64, bf16 output, 128-row aligned groups");
      return 1;
    }
  }
  if (fp4 && (h.K % 64 != 0 || h.out_f32 || (reinterpret_cast<uintptr_t>(h.w_scales) & 15) || (h.K / 16) % 16 != 0)) {
    snprintf(g_gemm_err, sizeof(g_gemm_err), "wgemm: NVFP4 weights need K %% 256 == 0, bf16 output, aligned scales");
    return 1;
  }
  // NVFP4: h.w = packed codes [rows, K / 2] bytes (row pitch h.ldw bytes), h.w_scales = e4m3 [rows, K / 16]
  const CUtensorMap* tmW = fp4 ? tmap_2d(h.w, uint64_t(h.w_rows), uint64_t(h.K / 2), uint64_t(h.ldw), BM, BK / 2, TM_U8, false)
                           : fp8 ? tmap_2d(h.w, uint64_t(h.w_rows), uint64_t(h.K), uint64_t(h.ldw), BM, 128, TM_U8, true)
                               : tmap_2d(h.w, uint64_t(h.w_rows), uint64_t(h.K), uint64_t(h.ldw) * 2, BM, BK, TM_BF16, true);
  const CUtensorMap* tmS = fp4 ? tmap_2d(h.w_scales, uint64_t(h.w_rows), uint64_t(h.K / 16), uint64_t(h.K / 16), BM, 16,
                                         TM_U8, false)
                               : tmW;
  const CUtensorMap* tmX =
      fp8 ? tmap_2d(h.x, uint64_t(h.x_rows), uint64_t(h.K), uint64_t(h.ldx), uint32_t(bn), 128, TM_U8, true)
          : tmap_2d(h.x, uint64_t(h.x_rows), uint64_t(h.x_cols > 0 ? h.x_cols : h.K), uint64_t(h.ldx) * 2, uint32_t(bn),
                    BK, TM_BF16, true);
  if (!tmW || !tmX || !tmS) {
    snprintf(g_gemm_err, sizeof(g_gemm_err), "wgemm: %s", tmap_last_error());
    return 1;
  }
  WgemmArgs a{};
  a.out = h.out; a.ldo = h.ldo; a.residual = h.residual; a.ldr = h.ldr;
  a.tok_scale = h.tok_scale; a.out_rows = h.out_rows;
  a.K = h.K; a.n_feat = h.n_feat; a.feat_tiles = (h.n_feat + BM - 1) / BM;
  a.n_tok = h.n_tok;
  a.comm = h.comm;
  a.head = h.head;
  a.w_gscale = h.w_gscale;
  a.w_bscale = h.w_bscale; a.x_bscale = h.x_bscale;
  a.q8_out = h.q8_out; a.q8_scale = h.q8_scale;
  if (h.q8_out && (!fp8 || !h.dual || !h.q8_scale || h.n_feat % 128 != 0 || h.out_f32 || h.out_rows || h.residual ||
                   h.tok_scale || h.n_out_peer > 0 || (reinterpret_cast<uintptr_t>(h.q8_out) & 7))) {
    snprintf(g_gemm_err, sizeof(g_gemm_err), "wgemm: the encoded output needs the FP8 gate/up form, n_feat %% 128 == 0, plain rows");
    return 1;
  }
  a.tile_group = h.tile_group; a.tile_tok0 = h.tile_tok0; a.tile_out0 = h.tile_out0; a.tile_ntok = h.tile_ntok; a.n_tiles_dev = h.n_tiles_dev;
  a.n_tok_tiles_max = h.n_tok_tiles_max;
  a.rows_per_group = h.rows_per_group; a.dual_offset = h.dual_offset;
  a.x_group_col = h.x_group_col;
  if (h.x_group_col != 0 && (h.x_group_col % 8 != 0 || h.K % BK != 0 || fp8 || fp4 || !h.tile_group)) {
    snprintf(g_gemm_err, sizeof(g_gemm_err),
             "wgemm: per-group activation columns need grouped bf16 mode, K %% 64 == 0 and 16-byte aligned offsets");
    return 1;
  }
  a.split_k = h.split_k < 1 ? 1 : h.split_k;
  a.ws = h.ws; a.counters = h.counters; a.status = h.status;
  a.n_out_peer = h.n_out_peer;
  for (int i = 0; i < 8; ++i) a.out_peer[i] = h.out_peer[i];
  a.vec_ok = (!h.out_f32 && h.n_feat % 8 == 0 && h.ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(h.out) & 15) == 0 &&
              (!h.residual || (h.ldr % 8 == 0 && (reinterpret_cast<uintptr_t>(h.residual) & 15) == 0)))
                 ? 1 : 0;
  if (h.q8_out) a.vec_ok = 1;     // the encoded rows always leave through the staged write-out
  const int num_kb = fp8 ? h.K / 128 : (h.K + BK - 1) / BK;
  if (a.split_k > num_kb) a.split_k = num_kb;
  while (a.split_k > 1 && (a.split_k - 1) * ((num_kb + a.split_k - 1) / a.split_k) >= num_kb) --a.split_k;
  if (a.split_k > 1 && (!a.ws || !a.counters)) {
    snprintf(g_gemm_err, sizeof(g_gemm_err), "wgemm: split-K needs a workspace and counters");
    return 1;
  }
  const int n_tok_tiles = h.tile_group ? h.n_tok_tiles_max : (h.n_tok + bn - 1) / bn;
  long total = long(n_tok_tiles) * a.feat_tiles * a.split_k;
  if (total <= 0) return 0;
  int grid = int(total < g_num_sms ? total : g_num_sms);

#define LB_CASE(BN_, DUAL_)                                                                     \
  if (bn == BN_ && h.dual == DUAL_) {                                                           \
    if (fp4) return launch<BN_, DUAL_, false, true>(tmW, tmX, tmS, a, grid, stream);            \
    if (fp8) {                                                                                  \
      if constexpr (BN_ <= 64) return launch<BN_, DUAL_, false, false, true>(tmW, tmX, tmS, a, grid, stream); \
    }                                                                                           \
    return h.out_f32 ? launch<BN_, DUAL_, true>(tmW, tmX, tmS, a, grid, stream)                 \
                     : launch<BN_, DUAL_, false>(tmW, tmX, tmS, a, grid, stream);               \
  }
  LB_CASE(32, false) LB_CASE(64, false) LB_CASE(128, false) LB_CASE(256, false)
  LB_CASE(32, true) LB_CASE(64, true) LB_CASE(128, true)
#undef LB_CASE
  snprintf(g_gemm_err, sizeof(g_gemm_err), "wgemm: unsupported tile bn=%d dual=%d", bn, int(h.dual));
  return 1;
}

}  // namespace lb
