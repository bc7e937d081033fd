// Device-side pieces of the symmetric-memory collectives, shared by the stand-alone kernels (comm.cu) and by the
// GEMM whose tail performs the reduction itself (gemm_sm100.cu): system-scope flag stores / loads, the bounded
// flag wait, and the rank-ordered row reduction with residual add and RMSNorm.
#pragma once
#include "comm.h"
#include "common.cuh"
#include "nvfp4_dev.cuh"

namespace lb {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Waits until *flag >= want (wrap-safe) or the deadline passes. Returns false on timeout. The clock is first read
// after 64 failed polls (a read of %globaltimer is slow enough to matter on a wait that is usually short).
__device__ __forceinline__ bool wait_flag_geq(const uint32_t* flag, uint32_t want, uint64_t budget_ns) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (int32_t(ld_acquire_sys(flag) - want) < 0) {
    if ((++spins & 0x3f) == 0) {
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget_ns) return false;
    }
  }
  return true;
}

// Rows [blockIdx.x, T) step gridDim.x of sum_r partial_r (+ residual), summed in rank order over peer loads (same
// bits on every rank), optionally followed by RMSNorm of the summed row. `red` is >= 32 floats of shared memory.
// Every thread of the block must call it (block-wide barriers inside).
template <class Load>
__device__ __forceinline__ void reduce_rows_with(const Load& load, int world, int T, int H,
                                                       const __nv_bfloat16* __restrict__ residual, long ldr,
                                                       __nv_bfloat16* __restrict__ sum_out, long lds,
                                                       const float* __restrict__ norm_w, float eps, float w_offset,
                                                       __nv_bfloat16* __restrict__ norm_out, long ldn, float* red,
                                                       const Nv4RowsOut q = Nv4RowsOut{}) {
  const int nv = H / 8;
  const int nthr = blockDim.x, nwarp = (blockDim.x + 31) >> 5;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    float ss = 0.f;
    for (int v = threadIdx.x; v < nv; v += nthr) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      // every rank's vector is requested before the first one is added (the sum still runs in rank order): with
      // the loads issued one after the other a thread waited one NVLink round trip per rank
      uint4 ur[LB_MAX_RANKS];
#pragma unroll
      for (int r = 0; r < LB_MAX_RANKS; ++r)
        if (r < world) ur[r] = load(r, row, v);
#pragma unroll
      for (int r = 0; r < LB_MAX_RANKS; ++r) {
        if (r < world) {
          const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&ur[r]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(u2[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
          }
        }
      }
      if (residual) {
        const uint4 u = reinterpret_cast<const uint4*>(residual + long(row) * ldr)[v];
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(u2[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      uint4 o;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        o2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        const float2 f = __bfloat1622float2(o2[j]);
        ss += f.x * f.x + f.y * f.y;
      }
      reinterpret_cast<uint4*>(sum_out + long(row) * lds)[v] = o;
    }
    if (norm_out) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
      __syncthreads();
      float tot = 0.f;
      for (int i = 0; i < nwarp; ++i) tot += red[i];
      const float inv = rsqrtf(tot / float(H) + eps);
      float amax = 0.f;
      for (int v = threadIdx.x; v < nv; v += nthr) {
        uint4 u = reinterpret_cast<const uint4*>(sum_out + long(row) * lds)[v];  // written by this thread above
        __nv_bfloat162* u2 = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(u2[j]);
          u2[j] = __floats2bfloat162_rn(f.x * inv * (norm_w[v * 8 + 2 * j] + w_offset),
                                        f.y * inv * (norm_w[v * 8 + 2 * j + 1] + w_offset));
          const float2 g = __bfloat1622float2(u2[j]);
          amax = fmaxf(amax, fmaxf(fabsf(g.x), fabsf(g.y)));
        }
        reinterpret_cast<uint4*>(norm_out + long(row) * ldn)[v] = u;
      }
      __syncthreads();
      if (q.codes) {
        // the normalised row once more as NVFP4 (row scale amax / (6 * 448), one UE4M3 scale per 16 values): the
        // expert GEMMs read this, the router reads the bf16 row
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
        __syncthreads();
        float m = 0.f;
        for (int i = 0; i < nwarp; ++i) m = fmaxf(m, red[i]);
        const float gs = fmaxf(m / (6.f * 448.f), 1e-12f);
        if (threadIdx.x == 0) q.row_gscale[row] = gs;
        for (int v = threadIdx.x; v < nv; v += nthr) {
          const uint4 u = reinterpret_cast<const uint4*>(norm_out + long(row) * ldn)[v];   // this thread's own write
          const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
          float f8[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(u2[j]);
            f8[2 * j] = f.x;
            f8[2 * j + 1] = f.y;
          }
          const uint32_t c = nv4_encode8_pair(f8, gs, q.sf, row, v * 8, q.k4, true);
          *reinterpret_cast<uint32_t*>(q.codes + long(row) * q.ld + v * 4) = c;
        }
        __syncthreads();
      }
    }
  }
}

// The plain form: rank r's vector is a peer load from its partial rows at buf_off of its symmetric buffer.
__device__ __forceinline__ void reduce_rows_rank_order(const CommPeers& peers, long buf_off, int T, int H,
                                                       const __nv_bfloat16* __restrict__ residual, long ldr,
                                                       __nv_bfloat16* __restrict__ sum_out, long lds,
                                                       const float* __restrict__ norm_w, float eps, float w_offset,
                                                       __nv_bfloat16* __restrict__ norm_out, long ldn, float* red,
                                                       const Nv4RowsOut q = Nv4RowsOut{}) {
  auto load = [&](int r, int row, int v) {
    return reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(peers.buffer[r]) + buf_off + (long(row) * H) * 2)[v];
  };
  reduce_rows_with(load, peers.world, T, H, residual, ldr, sum_out, lds, norm_w, eps, w_offset, norm_out, ldn, red, q);
}

}  // namespace lb
