// Native NVFP4 GEMM for sm_100a: e2m1 weights x e2m1 activations on the block-scaled tensor-core instruction
// (tcgen05.mma kind::mxf4nvf4, one UE4M3 scale per 16 elements on both operands), fp32 accumulation in TMEM.
//
//   out[token, feature] = w_gscale[group] * x_gscale[token] *
//                         sum_k (W[group * rows_per_group + feature, k] * sfW) * (X[token, k] * sfX)
//
// Same orientation and work decomposition as the bf16 GEMM (gemm_sm100.cu): weight rows are the UMMA M dimension
// (128 per tile), tokens the N dimension (32 / 64 / 128 accumulator columns), dense or grouped over a device-built
// list of (expert, token range) tiles, optional dual mode (gate and up tiles into two accumulators, SwiGLU in the
// epilogue). Nothing is expanded on the way: TMA streams the packed 4-bit codes (128 rows x 128 bytes = 256
// elements of K per stage, 128-byte swizzle) straight into the operand tiles, the scale factors of a stage come as
// one 2 KiB bulk copy per operand (see gemm_nvfp4_sm100.h for the atom layout), tcgen05.cp moves them into tensor
// memory and four MMAs of K = 64 consume the stage. A decode step therefore reads 0.56 bytes per weight.
//
// The epilogue can re-encode its result to NVFP4 (codes + scale atoms, static tensor scale) so that the SwiGLU
// output feeds the down projection without a bf16 round trip or a separate quantisation launch.
//
// Roles per CTA (192 threads, persistent over work items): warp 0 = TMA / bulk-copy producer, warp 1 = scale copy +
// MMA issuer (one thread), warps 2..5 = epilogue. Every wait is bounded and reports through the status word.
//
// Counterpart in the reference: src/cuda/sm120/nvfp4_a4.cu (mma.sync block-scaled FP4 for sm_120; quantiser,
// fused RMSNorm quantiser, grouped GEMM with SwiGLU and routing-weight epilogue).
#include <cuda_fp8.h>

#include "common.cuh"
#include "gemm_nvfp4_sm100.h"
#include "nvfp4_dev.cuh"
#include "tmap.cuh"

namespace lb {
namespace {

constexpr int BM = 128;                 // weight rows per tile
constexpr int KB_BYTES = 128;           // packed code bytes per row and stage (256 elements of K)
constexpr int W_TILE = BM * KB_BYTES;   // 16 KiB
constexpr int SF_TILE = 2048;           // four scale atoms: 128 rows x 256 elements
constexpr int SMEM_BUDGET = 200 * 1024;

constexpr int pow2_ge(int v) { return v <= 32 ? 32 : (v <= 64 ? 64 : (v <= 128 ? 128 : (v <= 256 ? 256 : 512))); }

// NCTA: sized for that many CTAs per SM (a share of the shared memory and tensor memory each). Short-K GEMMs are bound by the
// latency of their dependent hand-overs, not by bytes in flight, and a second CTA on the SM fills the gaps.
// EPI2: two epilogue warpgroups (warps 2..5 and 6..9), each with its own staging tile, on alternate 32-token column
// blocks of the accumulator: prompt-sized grouped GEMMs with short K (the down projection of an expert: two stages
// per tile) are bound by the epilogue, not by the main loop.
template <int BN, bool DUAL, int FT = 1, int NCTA = 1, bool EPI2 = false>
struct Cfg {
  static constexpr int NW = DUAL ? 2 : 1;
  static constexpr int X_TILE = BN * KB_BYTES;
  static constexpr int X_OFF = NW * W_TILE;
  static constexpr int SFW_OFF = X_OFF + X_TILE;
  static constexpr int SFX_OFF = SFW_OFF + NW * SF_TILE;
  static constexpr int STAGE_BYTES = SFX_OFF + SF_TILE;
  static constexpr int NSETS = EPI2 ? 2 : 1;
  static constexpr int BUDGET = NCTA == 1 ? (EPI2 ? SMEM_BUDGET - 16 * 1024 : SMEM_BUDGET) : (NCTA == 2 ? 94 * 1024 : 54 * 1024);
  static constexpr int STAGES_RAW = BUDGET / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int TMEM_MAX = NCTA == 1 ? 512 : (NCTA == 2 ? 256 : 128);
  // A work item is FT consecutive 128-feature tiles of one token tile, accumulated side by side in one TMEM
  // buffer and handed to the epilogue together: a tile of a short-K GEMM (K = 512: two stages) is too little work
  // per hand-over (measured ~1 us of fixed cost per work item in every role).
  static constexpr int SUB_COLS = BN * NW;              // accumulator columns of one 128-feature tile
  static constexpr int ACC_COLS = SUB_COLS * FT;
  static constexpr int NACC = (2 * ACC_COLS + NW * 16 + 16 <= TMEM_MAX) ? 2 : 1;
  static constexpr int SFA_COL = NACC * ACC_COLS;       // 16 columns per weight tile: 4 k steps x 4 row groups
  static constexpr int SFB_COL = SFA_COL + NW * 16;     // 16 columns for the token tile
  static constexpr int TMEM_COLS = pow2_ge(SFB_COL + 16);
  static constexpr int EPI_BYTES = NSETS * 32 * BM * 4;
  static constexpr int THREADS = 64 + 128 * NSETS;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 512;
  static_assert(STAGE_BYTES % 1024 == 0, "stages must keep the 1024-byte alignment of swizzled tiles");
  static_assert(SFB_COL + 16 <= TMEM_MAX, "accumulators and scale factors do not fit tensor memory");
  static_assert(STAGES >= 2, "too few stages");
};

struct Args {
  const uint8_t* w_sf; const uint8_t* x_sf;
  const float* w_gscale; const float* x_gscale; int x_gs_stride;
  __nv_bfloat16* out; long ldo;
  const __nv_bfloat16* residual; long ldr;
  const float* tok_scale; const int* out_rows;
  uint8_t* q_codes; long q_ld; uint8_t* q_sf; const float* q_gscale; int q_k4;
  int K, n_feat, feat_tiles, n_tok, k4;
  const int* tile_group; const int* tile_tok0; const int* tile_out0; const int* tile_ntok; const int* n_tiles_dev;
  int n_tok_tiles_max, rows_per_group, dual_offset, act, vec_ok;
  int* status;
};

struct Work { int group, tok0, out0, ntok, feat0; };

template <int BN, int FT>
__device__ __forceinline__ bool decode_work(const Args& a, int w, int n_tok_tiles, Work& it) {
  const int items = (a.feat_tiles + FT - 1) / FT;       // work items per token tile
  const int tt = w / items;
  if (tt >= n_tok_tiles) return false;
  it.feat0 = (w - tt * items) * (BM * FT);
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

// Shared-memory descriptor of one scale atom for tcgen05.cp: 32 rows of 16 bytes, no swizzle, 8-row groups
// 128 bytes apart.
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3ffff) >> 4);
  d |= uint64_t(128 >> 4) << 32;
  d |= uint64_t(1) << 46;
  return d;
}
__device__ __forceinline__ void sf_copy(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma_nvf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
// Instruction descriptor: e2m1 x e2m1, UE4M3 scales, K-major operands, fp32 accumulate, K = 64.
__host__ __device__ constexpr uint32_t nvf4_idesc(uint32_t M, uint32_t N) {
  return (1u << 7) | (1u << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

template <int BN, bool DUAL, bool QOUT, int FT, int NCTA, bool EPI2>
__global__ void __launch_bounds__(EPI2 ? 320 : 192, NCTA)
wgemm_nv4_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const Args a) {
  using C = Cfg<BN, DUAL, FT, NCTA, EPI2>;
  constexpr int STAGES = C::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* stage = reinterpret_cast<float*>(smem + STAGES * C::STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * C::STAGE_BYTES + C::EPI_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = bars + 2 * STAGES + C::NACC;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * C::NACC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < C::NACC; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4 * C::NSETS);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  griddep_wait();
  griddep_launch();

  const int n_tok_tiles = a.tile_group ? min(*a.n_tiles_dev, a.n_tok_tiles_max) : (a.n_tok + BN - 1) / BN;
  const int num_kb = (a.K + 255) / 256;            // stages per tile
  const int k_steps_last = ((a.K - (num_kb - 1) * 256) + 63) / 64;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      tma_prefetch_desc(&tmW);
      tma_prefetch_desc(&tmX);
      int s = 0;
      uint32_t ph = 0;
      int issued = 0;
      bool ok = true;
      // the next item's table entries are fetched while the current one is processed (every role does this)
      Work it, nx;
      bool have = decode_work<BN, FT>(a, blockIdx.x, n_tok_tiles, it);
      for (int w = blockIdx.x; ok && have; w += gridDim.x, it = nx) {
        have = decode_work<BN, FT>(a, w + gridDim.x, n_tok_tiles, nx);
        const uint8_t* sfx = a.x_sf + long(it.tok0 >> 7) * a.k4 * 512;
        for (int f = 0; ok && f < FT; ++f) {
          if (it.feat0 + f * BM >= a.n_feat) break;
          const int wrow = it.group * a.rows_per_group + it.feat0 + f * BM;
          const uint8_t* sfw = a.w_sf + long(wrow >> 7) * a.k4 * 512;
          const uint8_t* sfw2 = DUAL ? a.w_sf + long((wrow + a.dual_offset) >> 7) * a.k4 * 512 : nullptr;
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) {
              *abort_flag = 1;
              atomicCAS(a.status, 0, ST_TIMEOUT_EMPTY);
              ok = false;
              break;
            }
            uint8_t* st = smem + s * C::STAGE_BYTES;
            mbar_expect_tx(&full[s], C::STAGE_BYTES);
            tma_load_2d(st, &tmW, &full[s], kb * KB_BYTES, wrow);
            if (DUAL) tma_load_2d(st + W_TILE, &tmW, &full[s], kb * KB_BYTES, wrow + a.dual_offset);
            tma_load_2d(st + C::X_OFF, &tmX, &full[s], kb * KB_BYTES, it.tok0);
            bulk_load(st + C::SFW_OFF, sfw + long(kb) * SF_TILE, SF_TILE, &full[s]);
            if (DUAL) bulk_load(st + C::SFW_OFF + SF_TILE, sfw2 + long(kb) * SF_TILE, SF_TILE, &full[s]);
            bulk_load(st + C::SFX_OFF, sfx + long(kb) * SF_TILE, SF_TILE, &full[s]);
            ++issued;
            if (++s == STAGES) { s = 0; ph ^= 1; }
          }
        }
      }
      if (!ok) {
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
    // ------------------------------------------------------------------ scale copies + MMA
    if (lane == 0) {
      constexpr uint32_t idesc = nvf4_idesc(BM, BN);
      const uint32_t sfa_t = tmem_base + C::SFA_COL;
      const uint32_t sfb_t = tmem_base + C::SFB_COL;
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      Work it, nx;
      bool have = decode_work<BN, FT>(a, blockIdx.x, n_tok_tiles, it);
      for (int w = blockIdx.x; ok && have; w += gridDim.x, it = nx) {
        have = decode_work<BN, FT>(a, w + gridDim.x, n_tok_tiles, nx);
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, abort_flag)) {
          *abort_flag = 1;
          atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_EMPTY);
          break;
        }
        tc_fence_after();
        // Row group of the token tile inside its 128-row scale atom = column offset of its scale factors. Only
        // offsets that are multiples of two columns are used (64-token tiles on 64-row boundaries); a 32-token
        // tile must start a 128-row atom. An odd column offset raised "misaligned address" on B200.
        const uint32_t grp = uint32_t((it.tok0 & 127) >> 5);
        if ((BN == 32 && grp != 0) || (BN == 64 && (grp & 1)) || (BN == 128 && grp != 0)) {
          *abort_flag = 1;
          atomicCAS(a.status, 0, ST_BAD_ARGS);
          break;
        }
        const uint32_t sfb_col = sfb_t + grp;
        for (int f = 0; ok && f < FT; ++f) {
          if (it.feat0 + f * BM >= a.n_feat) break;
          const uint32_t d0 = tmem_base + acc * C::ACC_COLS + f * C::SUB_COLS;
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait(&full[s], ph, abort_flag)) {
              *abort_flag = 1;
              atomicCAS(a.status, 0, ST_TIMEOUT_FULL);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + s * C::STAGE_BYTES);
            const int nk = kb == num_kb - 1 ? k_steps_last : 4;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              if (k < nk) {
                sf_copy(sfa_t + k * 4, sf_desc(sa + C::SFW_OFF + k * 512));
                if (DUAL) sf_copy(sfa_t + 16 + k * 4, sf_desc(sa + C::SFW_OFF + SF_TILE + k * 512));
                sf_copy(sfb_t + k * 4, sf_desc(sa + C::SFX_OFF + k * 512));
              }
            }
            const uint64_t dw = umma_desc_k_sw128(sa);
            const uint64_t dw2 = umma_desc_k_sw128(sa + W_TILE);
            const uint64_t dx = umma_desc_k_sw128(sa + C::X_OFF);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              if (k < nk) {
                const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
                const uint64_t koff = uint64_t(k * 2);            // 32 bytes of codes per K = 64 step
                umma_nvf4(d0, dw + koff, dx + koff, idesc, sfa_t + k * 4, sfb_col + k * 4, accum);
                if (DUAL) umma_nvf4(d0 + BN, dw2 + koff, dx + koff, idesc, sfa_t + 16 + k * 4, sfb_col + k * 4, accum);
              }
            }
            umma_commit(&empty[s]);
            if (++s == STAGES) { s = 0; ph ^= 1; }
          }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        if (++acc == C::NACC) { acc = 0; acc_ph ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, with EPI2 also 6..9)
    const int q = warp & 3;
    const int eset = (warp - 2) >> 2;                  // epilogue warpgroup: 32-token column blocks eset, eset + NSETS, ...
    const int etid = threadIdx.x - 64 - eset * 128;
    float* const stage_all = stage;
    float* stage = stage_all + eset * (32 * BM);
    int acc = 0;
    uint32_t acc_ph = 0;
    Work it, nx;
    const float q_gs = QOUT ? *a.q_gscale : 1.f;
    const float xs_all = (a.x_gscale && a.x_gs_stride == 0) ? __ldg(a.x_gscale) : 1.f;
    bool have = decode_work<BN, FT>(a, blockIdx.x, n_tok_tiles, it);
    for (int w = blockIdx.x; have; w += gridDim.x, it = nx) {
      have = decode_work<BN, FT>(a, w + gridDim.x, n_tok_tiles, nx);
      const int row = q * 32 + lane;
      // Row bookkeeping of the first 32 token columns is fetched BEFORE the accumulator is waited for, so these
      // (dependent, L2-latency) loads overlap the tile's MMAs instead of sitting between them and the stores:
      // the output row and routing weight of the four rows this thread writes, the activation scale of column
      // `lane` (handed round by shuffles).
      long orow_p[4];
      float sc_p[4];
      float xs_lane = xs_all;
      auto prefetch_rows = [&](int c) {
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
          const int t = c + pass * 8 + (etid >> 4);
          const int xrow = it.out0 + t;
          orow_p[pass] = -1;
          sc_p[pass] = 1.f;
          if (!QOUT && t < it.ntok) {
            orow_p[pass] = a.out_rows ? long(a.out_rows[xrow]) : long(xrow);
            if (a.tok_scale) sc_p[pass] = a.tok_scale[xrow];
          }
        }
        if (a.x_gscale && a.x_gs_stride != 0)
          xs_lane = (c + lane < it.ntok) ? __ldg(&a.x_gscale[long(it.tok0 + c + lane) * a.x_gs_stride]) : 1.f;
      };
      prefetch_rows(eset * 32);
      if (!__all_sync(0xffffffffu, mbar_wait(&tfull[acc], acc_ph, abort_flag))) {
        *abort_flag = 1;
        atomicCAS(a.status, 0, ST_TIMEOUT_TMEM_FULL);
        break;
      }
      tc_fence_after();
      const float gs0 = a.w_gscale ? a.w_gscale[it.group * C::NW] : 1.f;
      const float gs1 = (DUAL && a.w_gscale) ? a.w_gscale[it.group * 2 + 1] : 1.f;
      const int item_feat0 = it.feat0;
#pragma unroll 1
      for (int f = 0; f < FT; ++f) {
      it.feat0 = item_feat0 + f * BM;
      if (it.feat0 >= a.n_feat) break;
      const uint32_t t0 = tmem_base + (uint32_t(q * 32) << 16) + acc * C::ACC_COLS + f * C::SUB_COLS;
#pragma unroll 1
      for (int c = eset * 32; c < BN; c += 32 * C::NSETS) {
        if (c >= it.ntok) break;
        if (c > eset * 32 || (f > 0 && BN > 32)) prefetch_rows(c);
        uint32_t r[32];
        float g[32];
        tmem_ld32(t0 + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) g[j] = __uint_as_float(r[j]);
        if (DUAL) {
          tmem_ld32(t0 + BN + c, r);
          tmem_ld_wait();
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float xs = __shfl_sync(0xffffffffu, xs_lane, j);
          float v = g[j] * gs0 * xs;
          if (DUAL) {
            const float u = __uint_as_float(r[j]) * gs1 * xs;
            if (a.act == 0) v = (v / (1.f + __expf(-v))) * u;
            else v = 0.5f * v * (1.f + tanhf(0.7978845608f * (v + 0.044715f * v * v * v))) * u;
          }
          stage[j * BM + row] = v;
        }
        if (eset == 0) asm volatile("bar.sync 2, 128;" ::: "memory");
        else asm volatile("bar.sync 3, 128;" ::: "memory");
        const int f8 = (etid & 15) * 8;
        const int feat8 = it.feat0 + f8;
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
          const int j = pass * 8 + (etid >> 4);
          const int t = c + j;
          const bool live = t < it.ntok && feat8 < a.n_feat;
          const float4 v0 = *reinterpret_cast<const float4*>(&stage[j * BM + f8]);
          const float4 v1 = *reinterpret_cast<const float4*>(&stage[j * BM + f8 + 4]);
          float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
          const int xrow = it.out0 + t;
          if (QOUT) {
            // 16 features = this thread and its neighbour: one scale byte, two words of codes
            float amax = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            const uint32_t sb = e4m3_enc(amax / (6.f * q_gs));
            const float sdec = e4m3_dec(sb) * q_gs;
            const float inv = sdec > 0.f ? 1.f / sdec : 0.f;
            if (live) {
              *reinterpret_cast<uint32_t*>(a.q_codes + long(xrow) * a.q_ld + (feat8 >> 1)) = pack_e2m1x8(v, inv);
              if ((etid & 1) == 0) a.q_sf[sf_atom_byte(xrow, feat8 >> 4, a.q_k4)] = uint8_t(sb);
            }
          } else if (live) {
            const long orow = orow_p[pass];
            if (orow >= 0) {
              const float sc = sc_p[pass];
#pragma unroll
              for (int e = 0; e < 8; ++e) v[e] *= sc;
              if (a.vec_ok) {
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
                *reinterpret_cast<uint4*>(a.out + orow * a.ldo + feat8) = o;
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  if (feat8 + e < a.n_feat) {
                    float o = v[e];
                    if (a.residual) o += __bfloat162float(a.residual[orow * a.ldr + feat8 + e]);
                    a.out[orow * a.ldo + feat8 + e] = __float2bfloat16(o);
                  }
                }
              }
            }
          }
        }
        if (eset == 0) asm volatile("bar.sync 2, 128;" ::: "memory");
        else asm volatile("bar.sync 3, 128;" ::: "memory");
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (++acc == C::NACC) { acc = 0; acc_ph ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

thread_local char g_err[512];
int g_sms = 0;

template <int BN, bool DUAL, bool QOUT, int FT, int NCTA = 1, bool EPI2 = false>
int launch(const CUtensorMap* tmW, const CUtensorMap* tmX, const Args& a, int grid, cudaStream_t stream) {
  using C = Cfg<BN, DUAL, FT, NCTA, EPI2>;
  auto kfn = wgemm_nv4_kernel<BN, DUAL, QOUT, FT, NCTA, EPI2>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) {
      snprintf(g_err, sizeof(g_err), "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return 1;
    }
    attr_set = true;
  }
  launch_pdl(kfn, dim3(grid), dim3(C::THREADS), C::SMEM_BYTES, stream, *tmW, *tmX, a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(g_err, sizeof(g_err), "wgemm_nv4 launch: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

}  // namespace

const char* wgemm_nv4_last_error() { return g_err; }

int wgemm_nv4_launch(const Nv4Host& h, cudaStream_t stream) {
  const bool qout = h.q_codes != nullptr;
  if (h.K % 64 != 0 || h.K <= 0 || (h.ldw % 16) || (h.ldx % 16) ||
      ((reinterpret_cast<uintptr_t>(h.w) | reinterpret_cast<uintptr_t>(h.x) | reinterpret_cast<uintptr_t>(h.w_sf) |
        reinterpret_cast<uintptr_t>(h.x_sf)) & 15)) {
    snprintf(g_err, sizeof(g_err), "wgemm_nv4: K must be a multiple of 64, pitches and bases 16-byte aligned");
    return 1;
  }
  if (h.rows_per_group % 128 != 0 || (h.dual && h.dual_offset % 128 != 0)) {
    snprintf(g_err, sizeof(g_err), "wgemm_nv4: groups (and the gate / up halves) must start on 128-row boundaries");
    return 1;
  }
  if (qout && (h.n_feat % 16 != 0 || !h.q_sf || !h.q_gscale || (h.q_ld % 4) || h.out_rows || h.tok_scale || h.residual)) {
    snprintf(g_err, sizeof(g_err), "wgemm_nv4: a quantised output needs n_feat %% 16 == 0 and no row map / scale / residual");
    return 1;
  }
  if (!h.tile_group && h.bn == 32 && h.n_tok > 32) {
    snprintf(g_err, sizeof(g_err), "wgemm_nv4: 32-token tiles serve up to 32 tokens (their scale factors must start a "
                                   "128-row atom); use 64 or 128");
    return 1;
  }
  if (!qout && !h.out) {
    snprintf(g_err, sizeof(g_err), "wgemm_nv4: no output");
    return 1;
  }
  if (g_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_sms <= 0) g_sms = 148;
  }
  const int bn = h.bn;
  const CUtensorMap* tmW = tmap_2d(h.w, uint64_t(h.w_rows), uint64_t(h.K / 2), uint64_t(h.ldw), BM, KB_BYTES, TM_U8, true);
  const CUtensorMap* tmX = tmap_2d(h.x, uint64_t(h.x_rows), uint64_t(h.K / 2), uint64_t(h.ldx), uint32_t(bn), KB_BYTES,
                                   TM_U8, true);
  if (!tmW || !tmX) {
    snprintf(g_err, sizeof(g_err), "wgemm_nv4: %s", tmap_last_error());
    return 1;
  }
  Args a{};
  a.w_sf = h.w_sf; a.x_sf = h.x_sf; a.w_gscale = h.w_gscale; a.x_gscale = h.x_gscale; a.x_gs_stride = h.x_gs_stride;
  a.out = static_cast<__nv_bfloat16*>(h.out); a.ldo = h.ldo; a.residual = h.residual; a.ldr = h.ldr;
  a.tok_scale = h.tok_scale; a.out_rows = h.out_rows;
  a.q_codes = h.q_codes; a.q_ld = h.q_ld; a.q_sf = h.q_sf; a.q_gscale = h.q_gscale; a.q_k4 = nv4_sf_k4(h.n_feat);
  a.K = h.K; a.n_feat = h.n_feat; a.feat_tiles = (h.n_feat + BM - 1) / BM; a.n_tok = h.n_tok; a.k4 = nv4_sf_k4(h.K);
  a.tile_group = h.tile_group; a.tile_tok0 = h.tile_tok0; a.tile_out0 = h.tile_out0; a.tile_ntok = h.tile_ntok;
  a.n_tiles_dev = h.n_tiles_dev; a.n_tok_tiles_max = h.n_tok_tiles_max;
  a.rows_per_group = h.rows_per_group; a.dual_offset = h.dual_offset; a.act = h.act;
  a.status = h.status;
  a.vec_ok = (!qout && h.n_feat % 8 == 0 && h.ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(h.out) & 15) == 0 &&
              (!h.residual || (h.ldr % 8 == 0 && (reinterpret_cast<uintptr_t>(h.residual) & 15) == 0))) ? 1 : 0;
  const int n_tok_tiles = h.tile_group ? h.n_tok_tiles_max : (h.n_tok + bn - 1) / bn;
  // Feature tiles per work item: short-K GEMMs with many feature tiles (the down projection of an expert: K = 512,
  // 16 tiles) take four at a time, the gate / up pair two; everything else one.
  const int num_kb = (h.K + 255) / 256;
  // Decode-sized grouped GEMMs are bound by the latency of their dependent hand-overs (TMA -> MMA thread -> commit ->
  // producer), not by bytes in flight: several CTAs per SM, each with a share of the shared memory and tensor
  // memory, fill the gaps. Measured on the 80B-A3B expert shapes at 16 tokens: gate/up 43 -> 34 us with two CTAs
  // per SM, down (K = 512: two stages per tile) 31 -> 22 -> 20 us with two / three.
  const bool short_k = bn == 32 && !h.dual && !qout && num_kb <= 4 && a.feat_tiles >= 8;
  const bool many_dual = bn == 32 && h.dual && qout && long(n_tok_tiles) * a.feat_tiles >= 2L * g_sms;
  const int ncta = short_k ? 3 : (many_dual ? 2 : 1);
  const int ft = 1;
  const long total = long(n_tok_tiles) * ((a.feat_tiles + ft - 1) / ft);
  if (total <= 0) return 0;
  const int slots = ncta * g_sms;
  const int grid = int(total < slots ? total : slots);
  // prompt-sized grouped steps with 64-token tiles: two epilogue warpgroups
  const bool big = h.tile_group && bn == 64 && h.n_tok_tiles_max >= 256;
  if (big && !h.dual && !qout) return launch<64, false, false, 1, 1, true>(tmW, tmX, a, grid, stream);
  if (big && h.dual && qout) return launch<64, true, true, 1, 1, true>(tmW, tmX, a, grid, stream);
  if (short_k) return launch<32, false, false, 1, 3>(tmW, tmX, a, grid, stream);
  if (many_dual) return launch<32, true, true, 1, 2>(tmW, tmX, a, grid, stream);
#define LB_NV4(BN_, DUAL_, FT_)                                                             \
  if (bn == BN_ && h.dual == DUAL_ && ft == FT_)                                            \
    return qout ? launch<BN_, DUAL_, true, FT_>(tmW, tmX, a, grid, stream)                  \
                : launch<BN_, DUAL_, false, FT_>(tmW, tmX, a, grid, stream);
  LB_NV4(32, false, 1) LB_NV4(64, false, 1) LB_NV4(128, false, 1) LB_NV4(32, true, 1) LB_NV4(64, true, 1)
  LB_NV4(128, true, 1)
#undef LB_NV4
  snprintf(g_err, sizeof(g_err), "wgemm_nv4: unsupported tile bn=%d dual=%d", bn, int(h.dual));
  return 1;
}

// ------------------------------------------------------------------------------------------------
// scale layout conversion
// ------------------------------------------------------------------------------------------------
namespace {

__global__ void pack_scales_kernel(const uint8_t* __restrict__ lin, long rows, long K, int k4, uint8_t* __restrict__ atoms,
                                   bool unpack, uint8_t* __restrict__ lin_out) {
  const long nb = K / 16;
  const long i = long(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows * nb) return;
  const long r = i / nb;
  const int b = int(i % nb);
  const long off = sf_atom_byte(r, b, k4);
  if (unpack) lin_out[i] = atoms[off];
  else atoms[off] = lin[i];
}

// One CTA per row, 128 threads; thread i owns the 16-element blocks i, i + 128, ...
__global__ void __launch_bounds__(128) act_quant_kernel(const __nv_bfloat16* __restrict__ x, long ldx,
                                                        const __nv_bfloat16* __restrict__ residual, long ldr,
                                                        __nv_bfloat16* __restrict__ sum_out, long lds,
                                                        const float* __restrict__ norm_w, float eps, float w_offset,
                                                        __nv_bfloat16* __restrict__ normed_out, long ldn, long K, int k4,
                                                        const float* __restrict__ gscale_static,
                                                        uint8_t* __restrict__ codes, long ldc, uint8_t* __restrict__ sf,
                                                        float* __restrict__ row_gscale) {
  constexpr int MAXB = 4;                 // blocks per thread: K <= 8192
  griddep_wait();
  griddep_launch();
  const long r = blockIdx.x;
  const int nb = int(K / 16);
  __shared__ float red[4];
  __shared__ float bcast;
  float v[MAXB][16];
  float ss = 0.f, amax = 0.f;
#pragma unroll
  for (int i = 0; i < MAXB; ++i) {
    const int b = threadIdx.x + i * 128;
    if (b < nb) {
      const uint4* p = reinterpret_cast<const uint4*>(x + r * ldx + b * 16);
      uint4 u[2] = {p[0], p[1]};
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(u);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float2 f = __bfloat1622float2(h2[e]);
        v[i][2 * e] = f.x;
        v[i][2 * e + 1] = f.y;
      }
      if (residual) {
        const uint4* pr = reinterpret_cast<const uint4*>(residual + r * ldr + b * 16);
        uint4 ur[2] = {pr[0], pr[1]};
        const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(ur);
        uint4 us[2];
        __nv_bfloat162* s2 = reinterpret_cast<__nv_bfloat162*>(us);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float2 f = __bfloat1622float2(r2[e]);
          s2[e] = __floats2bfloat162_rn(v[i][2 * e] + f.x, v[i][2 * e + 1] + f.y);
          const float2 g = __bfloat1622float2(s2[e]);
          v[i][2 * e] = g.x;
          v[i][2 * e + 1] = g.y;
        }
        if (sum_out) {
          uint4* po = reinterpret_cast<uint4*>(sum_out + r * lds + b * 16);
          po[0] = us[0];
          po[1] = us[1];
        }
      }
#pragma unroll
      for (int e = 0; e < 16; ++e) ss += v[i][e] * v[i][e];
    }
  }
  if (norm_w) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float inv = rsqrtf((red[0] + red[1] + red[2] + red[3]) / float(K) + eps);
    __syncthreads();
#pragma unroll
    for (int i = 0; i < MAXB; ++i) {
      const int b = threadIdx.x + i * 128;
      if (b < nb) {
        uint4 un[2];
        __nv_bfloat162* n2 = reinterpret_cast<__nv_bfloat162*>(un);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          n2[e] = __floats2bfloat162_rn(v[i][2 * e] * inv * (norm_w[b * 16 + 2 * e] + w_offset),
                                        v[i][2 * e + 1] * inv * (norm_w[b * 16 + 2 * e + 1] + w_offset));
          const float2 g = __bfloat1622float2(n2[e]);
          v[i][2 * e] = g.x;
          v[i][2 * e + 1] = g.y;
        }
        if (normed_out) {
          uint4* po = reinterpret_cast<uint4*>(normed_out + r * ldn + b * 16);
          po[0] = un[0];
          po[1] = un[1];
        }
      }
    }
  }
  float gs;
  if (gscale_static) {
    gs = *gscale_static;
  } else {
#pragma unroll
    for (int i = 0; i < MAXB; ++i) {
      if (threadIdx.x + i * 128 < nb) {
#pragma unroll
        for (int e = 0; e < 16; ++e) amax = fmaxf(amax, fabsf(v[i][e]));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
      const float m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
      bcast = fmaxf(m / (6.f * 448.f), 1e-12f);
      row_gscale[r] = bcast;
    }
    __syncthreads();
    gs = bcast;
  }
#pragma unroll
  for (int i = 0; i < MAXB; ++i) {
    const int b = threadIdx.x + i * 128;
    if (b < nb) {
      float bm = 0.f;
#pragma unroll
      for (int e = 0; e < 16; ++e) bm = fmaxf(bm, fabsf(v[i][e]));
      const uint32_t sb = e4m3_enc(bm / (6.f * gs));
      const float sdec = e4m3_dec(sb) * gs;
      const float inv = sdec > 0.f ? 1.f / sdec : 0.f;
      float lo[8], hi[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) { lo[e] = v[i][e]; hi[e] = v[i][8 + e]; }
      uint2 o;
      o.x = pack_e2m1x8(lo, inv);
      o.y = pack_e2m1x8(hi, inv);
      *reinterpret_cast<uint2*>(codes + r * ldc + b * 8) = o;
      sf[sf_atom_byte(r, b, k4)] = uint8_t(sb);
    }
  }
}

// One warp per destination row: dst row i = source row rows[i] (codes, the row's scale bytes inside their atoms, the
// row scale). rows[i] < 0: a padding row, left as it is.
__global__ void __launch_bounds__(256) nv4_gather_kernel(const uint8_t* __restrict__ codes, long ldc,
                                                         const uint8_t* __restrict__ sf, const float* __restrict__ gs,
                                                         int K, int k4, const int* __restrict__ rows,
                                                         const int* __restrict__ n_rows, long max_rows,
                                                         uint8_t* __restrict__ dcodes, long ldd, uint8_t* __restrict__ dsf,
                                                         float* __restrict__ dgs) {
  const int lane = threadIdx.x & 31;
  const long n = n_rows ? min(long(*n_rows), max_rows) : max_rows;
  const int vec = K / 32;                        // 16-byte vectors of codes per row
  for (long i = long(blockIdx.x) * 8 + (threadIdx.x >> 5); i < n; i += long(gridDim.x) * 8) {
    const int t = rows[i];
    if (t < 0) continue;
    const uint4* s4 = reinterpret_cast<const uint4*>(codes + long(t) * ldc);
    uint4* d4 = reinterpret_cast<uint4*>(dcodes + i * ldd);
    for (int j = lane; j < vec; j += 32) d4[j] = s4[j];
    for (int a = lane; a < k4; a += 32)
      *reinterpret_cast<uint32_t*>(dsf + sf_atom_byte(i, a * 4, k4)) =
          *reinterpret_cast<const uint32_t*>(sf + sf_atom_byte(t, a * 4, k4));
    if (lane == 0 && gs) dgs[i] = gs[t];
  }
}

}  // namespace

int nv4_gather_rows_launch(const uint8_t* codes, long ldc, const uint8_t* sf, const float* row_gscale, long K,
                           const int* rows, const int* n_rows, long max_rows, uint8_t* dst_codes, long ldd,
                           uint8_t* dst_sf, float* dst_gscale, cudaStream_t s) {
  if (K % 64 || (ldc % 16) || (ldd % 16) || ((reinterpret_cast<uintptr_t>(codes) | reinterpret_cast<uintptr_t>(dst_codes)) & 15))
    return 1;
  if (max_rows <= 0) return 0;
  const long ctas = (max_rows + 7) / 8;
  nv4_gather_kernel<<<unsigned(ctas < 8192 ? ctas : 8192), 256, 0, s>>>(codes, ldc, sf, row_gscale, int(K), nv4_sf_k4(K),
                                                                       rows, n_rows, max_rows, dst_codes, ldd, dst_sf,
                                                                       dst_gscale);
  return cudaGetLastError() != cudaSuccess;
}

int nv4_pack_scales_launch(const uint8_t* scales, long rows, long K, uint8_t* atoms, cudaStream_t s) {
  if (K % 16) return 1;
  const long n = rows * (K / 16);
  if (n <= 0) return 0;
  pack_scales_kernel<<<unsigned((n + 255) / 256), 256, 0, s>>>(scales, rows, K, nv4_sf_k4(K), atoms, false, nullptr);
  return cudaGetLastError() != cudaSuccess;
}

int nv4_unpack_scales_launch(const uint8_t* atoms, long rows, long K, uint8_t* scales, cudaStream_t s) {
  if (K % 16) return 1;
  const long n = rows * (K / 16);
  if (n <= 0) return 0;
  pack_scales_kernel<<<unsigned((n + 255) / 256), 256, 0, s>>>(nullptr, rows, K, nv4_sf_k4(K),
                                                               const_cast<uint8_t*>(atoms), true, scales);
  return cudaGetLastError() != cudaSuccess;
}

int nv4_act_quant_launch(const void* x, long ldx, const void* residual, long ldr, void* sum_out, long lds,
                         const float* norm_w, float eps, float w_offset, void* normed_out, long ldn, long rows, long K,
                         const float* gscale_static, uint8_t* codes, long ldc, uint8_t* sf_atoms, float* row_gscale,
                         cudaStream_t s) {
  if (K % 16 || K > 8192 || (ldx % 8) || (ldc % 8) || (residual && ldr % 8) || (sum_out && lds % 8) ||
      (normed_out && ldn % 8) || (!gscale_static && !row_gscale))
    return 1;
  if (rows <= 0) return 0;
  launch_pdl(act_quant_kernel, dim3(unsigned(rows)), dim3(128), 0, s, static_cast<const __nv_bfloat16*>(x), ldx,
             static_cast<const __nv_bfloat16*>(residual), ldr, static_cast<__nv_bfloat16*>(sum_out), lds, norm_w, eps,
             w_offset, static_cast<__nv_bfloat16*>(normed_out), ldn, K, nv4_sf_k4(K), gscale_static, codes, ldc,
             sf_atoms, row_gscale);
  return cudaGetLastError() != cudaSuccess;
}

}  // namespace lb
