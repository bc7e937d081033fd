// Device-side communication primitives over symmetric (peer-mapped) memory on NVLink / NVSwitch.
//
//   * signal / wait: per-source sequence flags in each rank's signal pad, system-scope release and
//     acquire, every wait bounded by a %globaltimer deadline that raises a status word instead of
//     hanging the stream.
//   * all_reduce_fused: one-shot all-reduce for decode-sized rows. Every rank has written its partial
//     into its own symmetric buffer (the GEMM epilogue writes there directly); the kernel signals,
//     waits for all peers, sums the peers' rows IN RANK ORDER with plain peer loads (same bits on
//     every rank), and optionally adds the residual and applies the next RMSNorm in the same pass.
//   * reduce_scatter_fused / all_gather_copy: the two halves of the two-shot form for large rows.
//
// Counterparts in the reference: src/cuda/pair_link.cu, src/cuda/glm_exchange.cu, src/cuda/tp_net.cu
// (tp_sum in rank order, all_reduce_add_norm).
#include "comm.h"

#include "comm_dev.cuh"
#include "common.cuh"

namespace lb {

// Entry of a collective kernel: the sequence number is DATA (read from *seq_ptr, so a captured CUDA
// graph can be replayed), block 0 raises this rank's flag on every peer, and every CTA waits until all
// peers have raised theirs. Returns false (status word set) when a peer did not show up in time.
__device__ __forceinline__ bool comm_enter(const CommPeers& peers, int slot_base, const uint32_t* seq_ptr,
                                           uint64_t budget_ns, int* status, int* s_ok, uint32_t* seq_out) {
  const uint32_t seq = *reinterpret_cast<const volatile uint32_t*>(seq_ptr) + 1;
  if (threadIdx.x < peers.world && blockIdx.x == 0) {
    uint32_t* remote = reinterpret_cast<uint32_t*>(peers.signal[threadIdx.x]) + slot_base + peers.rank;
    __threadfence_system();
    st_release_sys(remote, seq);
  }
  if (threadIdx.x == 0) *s_ok = 1;
  __syncthreads();
  if (threadIdx.x < peers.world) {
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(peers.signal[peers.rank]) + slot_base + threadIdx.x;
    if (!wait_flag_geq(mine, seq, budget_ns)) {
      *s_ok = 0;
      atomicCAS(status, 0, ST_TIMEOUT_FLAG);
    }
  }
  __syncthreads();
  *seq_out = seq;
  return *s_ok != 0;
}
// Exit: the last CTA to finish publishes the new sequence number (all CTAs have read the old one).
__device__ __forceinline__ void comm_exit(uint32_t* seq_ptr, unsigned int* done_ctr, uint32_t seq) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int old = atomicAdd(done_ctr, 1u);
    if (old == gridDim.x - 1) {
      *done_ctr = 0;
      *reinterpret_cast<volatile uint32_t*>(seq_ptr) = seq;
    }
  }
}

// A kernel whose only job is the bounded wait: used by the failure-detection test (a flag that
// nothing sets must end with ST_TIMEOUT_FLAG in the status word and a live context).
__global__ void wait_flag_kernel(const uint32_t* flag, uint32_t want, uint64_t budget_ns, int* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    if (!wait_flag_geq(flag, want, budget_ns)) atomicCAS(status, 0, ST_TIMEOUT_FLAG);
  }
}

int wait_flag_launch(const uint32_t* flag, uint32_t want, uint64_t budget_ns, int* status, cudaStream_t s) {
  wait_flag_kernel<<<1, 32, 0, s>>>(flag, want, budget_ns, status);
  return cudaGetLastError() != cudaSuccess;
}

// Barrier across ranks: write seq into slot [my_rank] of every peer's pad, wait for all slots of mine.
__global__ void barrier_kernel(CommPeers peers, int slot_base, uint32_t seq, uint64_t budget_ns, int* status) {
  const int r = threadIdx.x;
  if (r < peers.world) {
    uint32_t* remote = reinterpret_cast<uint32_t*>(peers.signal[r]) + slot_base + peers.rank;
    __threadfence_system();
    st_release_sys(remote, seq);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(peers.signal[peers.rank]) + slot_base + r;
    if (!wait_flag_geq(mine, seq, budget_ns)) atomicCAS(status, 0, ST_TIMEOUT_FLAG);
  }
}

int barrier_launch(const CommPeers& peers, int slot_base, uint32_t seq, uint64_t budget_ns, int* status,
                   cudaStream_t s) {
  barrier_kernel<<<1, 32, 0, s>>>(peers, slot_base, seq, budget_ns, status);
  return cudaGetLastError() != cudaSuccess;
}

// One CTA per row (grid-stride). buf_off: byte offset of the partial rows inside every rank's
// symmetric buffer; rows are [T, H] bf16 with pitch H.
__global__ void __launch_bounds__(256) all_reduce_fused_kernel(CommPeers peers, long buf_off, int slot_base,
                                                               uint32_t* seq_ptr, unsigned int* done_ctr, int T, int H,
                                                               const __nv_bfloat16* __restrict__ residual, long ldr,
                                                               __nv_bfloat16* __restrict__ sum_out, long lds,
                                                               const float* __restrict__ norm_w, float eps,
                                                               float w_offset, __nv_bfloat16* __restrict__ norm_out,
                                                               long ldn, uint64_t budget_ns, int* status,
                                                               const Nv4RowsOut q) {
  __shared__ int s_ok;
  __shared__ float red[32];
  uint32_t seq;
  const bool entered = comm_enter(peers, slot_base, seq_ptr, budget_ns, status, &s_ok, &seq);
  if (!entered) { comm_exit(seq_ptr, done_ctr, seq); return; }
  reduce_rows_rank_order(peers, buf_off, T, H, residual, ldr, sum_out, lds, norm_w, eps, w_offset, norm_out, ldn, red, q);
  comm_exit(seq_ptr, done_ctr, seq);
}

int all_reduce_fused_launch(const CommPeers& peers, long buf_off, int slot_base, uint32_t* seq_ptr, unsigned int* done_ctr, int T,
                            int H, const void* residual, long ldr, void* sum_out, long lds, const float* norm_w, float eps,
                            float w_offset, void* norm_out, long ldn, uint64_t budget_ns, int* status,
                            cudaStream_t s, const Nv4RowsOut& q) {
  if (T <= 0) return 0;
  if (H % 8 || peers.world > LB_MAX_RANKS) return 1;
  if (q.codes && (!norm_out || H % 256 || !q.sf || !q.row_gscale || (q.ld % 4))) return 1;
  const int grid = T < 1184 ? T : 1184;     // rows in flight: up to eight CTAs per SM
  all_reduce_fused_kernel<<<grid, 256, 0, s>>>(peers, buf_off, slot_base, seq_ptr, done_ctr, T, H,
                                               static_cast<const __nv_bfloat16*>(residual), ldr,
                                               static_cast<__nv_bfloat16*>(sum_out), lds, norm_w, eps, w_offset,
                                               static_cast<__nv_bfloat16*>(norm_out), ldn, budget_ns, status, q);
  return cudaGetLastError() != cudaSuccess;
}

// Decode-sized all-reduce with the data pushed, flag and payload in one store (the "low latency" line format:
// every 8 bytes carry 4 bytes of payload and the 4-byte sequence number, and an 8-byte store arrives whole). Each
// CTA owns a row: it reads this rank's partial row, stores it as such lines into its region of every peer's
// staging area, then polls its own staging area until the lines of all peers carry this call's sequence number
// and sums them in rank order. One NVLink crossing instead of three (flag, load request, load reply), no fences.
// Two staging areas alternate with the sequence number: a peer can write call n + 2's lines only after it has
// finished call n + 1, for which it needed this rank's lines of call n + 1, sent after call n was read.
__device__ __forceinline__ void st_ll(uint4* p, uint32_t a, uint32_t b, uint32_t flag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(flag), "r"(b), "r"(flag) : "memory");
}
__device__ __forceinline__ uint4 ld_ll(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(256) all_reduce_ll_kernel(CommPeers peers, long buf_off, long ll_off, int ll_rows,
                                                            uint32_t* seq_ptr, unsigned int* done_ctr, int T, int H,
                                                            const __nv_bfloat16* __restrict__ residual, long ldr,
                                                            __nv_bfloat16* __restrict__ sum_out, long lds,
                                                            const float* __restrict__ norm_w, float eps, float w_offset,
                                                            __nv_bfloat16* __restrict__ norm_out, long ldn,
                                                            uint64_t budget_ns, int* status, const Nv4RowsOut q,
                                                            const CombineSrc cs) {
  __shared__ float red[32];
  __shared__ int s_on[32];
  griddep_wait();
  griddep_launch();
  const uint32_t seq = *reinterpret_cast<const volatile uint32_t*>(seq_ptr) + 1;
  const int nv = H / 8;
  const int me = peers.rank, world = peers.world;
  const long area = long(ll_rows) * H * 4;                       // one source rank's lines: 2 x the payload
  const long par_off = ll_off + long(seq & 1u) * world * area;
  const char* mine = reinterpret_cast<const char*>(peers.buffer[me]);
  // push: this rank's partial rows into region `me` of every peer
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    if (cs.y) {
      __syncthreads();
      if (threadIdx.x < cs.k) {
        const int e = cs.ids[long(row) * cs.k + threadIdx.x];
        s_on[threadIdx.x] = (e >= cs.e_lo && e < cs.e_hi);
      }
      __syncthreads();
    }
    for (int v = threadIdx.x; v < nv; v += blockDim.x) {
      uint4 d;
      if (cs.y) {
        // this rank's partial row = its experts' weighted rows of the token, in choice order, + the shared expert's
        const __nv_bfloat16* y = static_cast<const __nv_bfloat16*>(cs.y);
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int c0 = 0; c0 < cs.k; c0 += 4) {
          uint4 u[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            u[i] = make_uint4(0u, 0u, 0u, 0u);
            if (c0 + i < cs.k && s_on[c0 + i]) u[i] = reinterpret_cast<const uint4*>(y + (long(row) * cs.k + c0 + i) * cs.ldy)[v];
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u[i]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __bfloat1622float2(u2[j]);
              acc[2 * j] += f.x;
              acc[2 * j + 1] += f.y;
            }
          }
        }
        if (cs.shared) {
          const uint4 u = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(cs.shared) + long(row) * cs.lds)[v];
          const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(u2[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
          }
        }
        __nv_bfloat162* d2 = reinterpret_cast<__nv_bfloat162*>(&d);
#pragma unroll
        for (int j = 0; j < 4; ++j) d2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        // kept in the slot for this thread's own read in the rank-ordered sum below
        reinterpret_cast<uint4*>(const_cast<char*>(mine) + buf_off + (long(row) * H) * 2)[v] = d;
      } else {
        d = reinterpret_cast<const uint4*>(mine + buf_off + (long(row) * H) * 2)[v];
      }
      const long line = par_off + me * area + (long(row) * nv + v) * 32;
      for (int i = 1; i < world; ++i) {
        const int p = (me + i) % world;
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(peers.buffer[p]) + line);
        st_ll(dst, d.x, d.y, seq);
        st_ll(dst + 1, d.z, d.w, seq);
      }
    }
  }
  auto load = [&](int r, int row, int v) -> uint4 {
    if (r == me) return reinterpret_cast<const uint4*>(mine + buf_off + (long(row) * H) * 2)[v];
    const uint4* src = reinterpret_cast<const uint4*>(mine + par_off + r * area + (long(row) * nv + v) * 32);
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (true) {
      const uint4 a = ld_ll(src), b = ld_ll(src + 1);
      if (a.y == seq && a.w == seq && b.y == seq && b.w == seq) return make_uint4(a.x, a.z, b.x, b.z);
      if ((++spins & 0x3f) == 0) {
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > budget_ns) {
          atomicCAS(status, 0, ST_TIMEOUT_FLAG);
          return make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
  };
  reduce_rows_with(load, world, T, H, residual, ldr, sum_out, lds, norm_w, eps, w_offset, norm_out, ldn, red, q);
  comm_exit(seq_ptr, done_ctr, seq);
}

int all_reduce_ll_launch(const CommPeers& peers, long buf_off, long ll_off, int ll_rows, uint32_t* seq_ptr,
                         unsigned int* done_ctr, int T, int H, const void* residual, long ldr, void* sum_out, long lds,
                         const float* norm_w, float eps, float w_offset, void* norm_out, long ldn, uint64_t budget_ns,
                         int* status, cudaStream_t s, const Nv4RowsOut& q, const CombineSrc& cs) {
  if (T <= 0) return 0;
  if (H % 8 || peers.world > LB_MAX_RANKS || T > ll_rows || (ll_off % 32) || (buf_off % 16)) return 1;
  if (cs.y && (cs.k <= 0 || cs.k > 32 || !cs.ids || (cs.ldy % 8) || (cs.shared && cs.lds % 8))) return 1;
  if (q.codes && (!norm_out || H % 256 || !q.sf || !q.row_gscale || (q.ld % 4))) return 1;
  launch_pdl(all_reduce_ll_kernel, dim3(T), dim3(256), 0, s, peers, buf_off, ll_off, ll_rows, seq_ptr, done_ctr, T, H,
             static_cast<const __nv_bfloat16*>(residual), ldr, static_cast<__nv_bfloat16*>(sum_out), lds, norm_w, eps,
             w_offset, static_cast<__nv_bfloat16*>(norm_out), ldn, budget_ns, status, q, cs);
  return cudaGetLastError() != cudaSuccess;
}

// Vocabulary-split LM head: every rank holds the arg-max (value, global token id) of its slice of the vocabulary for
// each row; the ranks exchange these pairs as pushed flag-carrying lines (16 bytes per row and source) and each picks
// the global best (larger value, then lower token id), so the greedy token of a step needs neither the full logits
// nor a gather of them. One CTA, one thread per row (at most 1024 rows).
__global__ void __launch_bounds__(1024) argmax_exchange_kernel(CommPeers peers, long ax_off, int ax_rows, uint32_t* seq_ptr,
                                                               unsigned int* done_ctr, int rows,
                                                               const float* __restrict__ val, const int* __restrict__ idx,
                                                               int vocab_offset, int* __restrict__ picks,
                                                               uint64_t budget_ns, int* status) {
  griddep_wait();
  griddep_launch();
  const uint32_t seq = *reinterpret_cast<const volatile uint32_t*>(seq_ptr) + 1;
  const int me = peers.rank, world = peers.world;
  const long area = long(ax_rows) * 16;
  const long par_off = ax_off + long(seq & 1u) * world * area;
  const int row = threadIdx.x;
  if (row < rows) {
    const float v = val[row];
    const int gi = idx[row] + vocab_offset;
    for (int i = 1; i < world; ++i) {
      const int p = (me + i) % world;
      st_ll(reinterpret_cast<uint4*>(reinterpret_cast<char*>(peers.buffer[p]) + par_off + me * area + long(row) * 16),
            __float_as_uint(v), uint32_t(gi), seq);
    }
    float bv = v;
    int bi = gi;
    const char* mine = reinterpret_cast<const char*>(peers.buffer[me]);
    for (int r = 0; r < world; ++r) {
      if (r == me) continue;
      const uint4* src = reinterpret_cast<const uint4*>(mine + par_off + r * area + long(row) * 16);
      uint64_t t0 = 0;
      uint32_t spins = 0;
      while (true) {
        const uint4 a = ld_ll(src);
        if (a.y == seq && a.w == seq) {
          const float ov = __uint_as_float(a.x);
          const int oi = int(a.z);
          if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
          break;
        }
        if ((++spins & 0x3f) == 0) {
          const uint64_t now = globaltimer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > budget_ns) {
            atomicCAS(status, 0, ST_TIMEOUT_FLAG);
            break;
          }
        }
      }
    }
    picks[row] = bi;
  }
  comm_exit(seq_ptr, done_ctr, seq);
}

int argmax_exchange_launch(const CommPeers& peers, long ax_off, int ax_rows, uint32_t* seq_ptr, unsigned int* done_ctr,
                           int rows, const float* val, const int* idx, int vocab_offset, int* picks, uint64_t budget_ns,
                           int* status, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (rows > ax_rows || rows > 1024 || peers.world > LB_MAX_RANKS || (ax_off % 16)) return 1;
  const int threads = ((rows + 31) / 32) * 32;
  launch_pdl(argmax_exchange_kernel, dim3(1), dim3(threads), 0, s, peers, ax_off, ax_rows, seq_ptr, done_ctr, rows, val,
             idx, vocab_offset, picks, budget_ns, status);
  return cudaGetLastError() != cudaSuccess;
}

// Reduce-scatter half of the two-shot form: this rank sums rows [row0, row0 + n_rows) over all peers in
// rank order (+ residual), writing the reduced rows into its own symmetric buffer at out_off so the
// all-gather half can fetch them, and into sum_out when given.
__global__ void __launch_bounds__(256) reduce_scatter_kernel(CommPeers peers, long buf_off, long out_off,
                                                             int slot_base, uint32_t* seq_ptr, unsigned int* done_ctr, int row0,
                                                             int n_rows, int H,
                                                             const __nv_bfloat16* __restrict__ residual, long ldr,
                                                             uint64_t budget_ns, int* status, char* mc_base) {
  __shared__ int s_ok;
  uint32_t seq;
  const bool entered = comm_enter(peers, slot_base, seq_ptr, budget_ns, status, &s_ok, &seq);
  if (!entered) { comm_exit(seq_ptr, done_ctr, seq); return; }
  const int nv = H / 8;
  char* my = reinterpret_cast<char*>(peers.buffer[peers.rank]);
  for (long i = long(blockIdx.x) * 256 + threadIdx.x; i < long(n_rows) * nv; i += long(gridDim.x) * 256) {
    const int row = row0 + int(i / nv);
    const int v = int(i % nv);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    uint4 ur[LB_MAX_RANKS];
    const int n_src = mc_base ? 1 : peers.world;
    if (mc_base) {
      // NVLink multicast address of the same bytes on every rank: ONE load whose value is the sum over the ranks,
      // added inside the switch with fp32 accumulation (one crossing per element instead of world - 1)
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                   : "=r"(ur[0].x), "=r"(ur[0].y), "=r"(ur[0].z), "=r"(ur[0].w)
                   : "l"(mc_base + buf_off + long(row) * H * 2 + long(v) * 16)
                   : "memory");
    } else {
      // all ranks' vectors requested before the first is added (summed in rank order all the same)
#pragma unroll
      for (int r = 0; r < LB_MAX_RANKS; ++r)
        if (r < n_src)
          ur[r] = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(peers.buffer[r]) + buf_off +
                                                 long(row) * H * 2)[v];
    }
#pragma unroll
    for (int r = 0; r < LB_MAX_RANKS; ++r) {
      if (r < n_src) {
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
    for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    if (mc_base) {
      // one multicast store puts the reduced vector into EVERY rank's result region: the gather that follows only
      // reads local memory
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                   ::"l"(mc_base + out_off + long(row) * H * 2 + long(v) * 16), "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w)
                   : "memory");
    } else {
      reinterpret_cast<uint4*>(my + out_off + long(row) * H * 2)[v] = o;
    }
  }
  comm_exit(seq_ptr, done_ctr, seq);
}

int reduce_scatter_launch(const CommPeers& peers, long buf_off, long out_off, int slot_base, uint32_t* seq_ptr, unsigned int* done_ctr,
                          int row0, int n_rows, int H, const void* residual, long ldr, uint64_t budget_ns, int* status,
                          cudaStream_t s, void* mc_base) {
  if (H % 8 || peers.world > LB_MAX_RANKS) return 1;
  if (mc_base && ((buf_off | out_off) % 16)) return 1;
  long work = long(n_rows) * (H / 8);
  int grid = int((work + 255) / 256);
  if (grid < 1) grid = 1;
  if (grid > 592) grid = 592;
  reduce_scatter_kernel<<<grid, 256, 0, s>>>(peers, buf_off, out_off, slot_base, seq_ptr, done_ctr, row0, n_rows, H,
                                             static_cast<const __nv_bfloat16*>(residual), ldr, budget_ns, status,
                                             static_cast<char*>(mc_base));
  return cudaGetLastError() != cudaSuccess;
}

// All-gather half: after a signal round, copy every rank's rows [rows_per_rank * r, ...) from its
// symmetric buffer at src_off into the local dense output.
__global__ void __launch_bounds__(256) all_gather_kernel(CommPeers peers, long src_off, int slot_base, uint32_t* seq_ptr,
                                                         unsigned int* done_ctr, int T, int H, __nv_bfloat16* __restrict__ out, long ldo,
                                                         uint64_t budget_ns, int* status, int local_only) {
  __shared__ int s_ok;
  uint32_t seq;
  const bool entered = comm_enter(peers, slot_base, seq_ptr, budget_ns, status, &s_ok, &seq);
  if (!entered) { comm_exit(seq_ptr, done_ctr, seq); return; }
  const int nv = H / 8;
  const int per = (T + peers.world - 1) / peers.world;
  // four vectors per thread and round: their (peer) loads are all in flight before the first store
  const long total = long(T) * nv, stride = long(gridDim.x) * 256;
  for (long i0 = long(blockIdx.x) * 256 + threadIdx.x; i0 < total; i0 += 4 * stride) {
    uint4 u[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const long i = i0 + k * stride;
      if (i < total) {
        const int row = int(i / nv);
        const int v = int(i % nv);
        int owner = row / per;
        if (owner >= peers.world) owner = peers.world - 1;
        if (local_only) owner = peers.rank;        // the reduced rows were multicast into every rank's region
        u[k] = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(peers.buffer[owner]) + src_off +
                                              long(row) * H * 2)[v];
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const long i = i0 + k * stride;
      if (i < total) reinterpret_cast<uint4*>(out + long(i / nv) * ldo)[int(i % nv)] = u[k];
    }
  }
  comm_exit(seq_ptr, done_ctr, seq);
}

int all_gather_launch(const CommPeers& peers, long src_off, int slot_base, uint32_t* seq_ptr,
                      unsigned int* done_ctr, int T, int H, void* out,
                      long ldo, uint64_t budget_ns, int* status, cudaStream_t s, int local_only) {
  if (H % 8 || peers.world > LB_MAX_RANKS) return 1;
  long work = long(T) * (H / 8);
  int grid = int((work + 255) / 256);
  if (grid < 1) grid = 1;
  if (grid > 592) grid = 592;
  all_gather_kernel<<<grid, 256, 0, s>>>(peers, src_off, slot_base, seq_ptr, done_ctr, T, H, static_cast<__nv_bfloat16*>(out), ldo,
                                         budget_ns, status, local_only);
  return cudaGetLastError() != cudaSuccess;
}

}  // namespace lb
