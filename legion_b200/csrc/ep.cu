// Expert-parallel all-to-all: token dispatch and result combine over NVLink peer stores.
//
// Every rank holds its own tokens (data-parallel attention) and E / world whole experts. Per MoE layer:
//   1. ep_publish_counts  each rank writes its per-expert pair counts into every peer's count table
//                         (peer stores + release flags), waits for the others (bounded), and derives
//                         (a) where its rows of each expert start inside the owner's receive buffer -
//                         rows of one expert are ordered by source rank, then by (token, choice), so the
//                         layout is deterministic - and (b) the row count of each of its own experts.
//   2. ep_push            the routing plan's gather is fused with the dispatch: each sorted row is read
//                         from the local activations and stored straight into the owner's receive
//                         buffer together with (source rank, pair index) and the routing weight; the
//                         last CTA raises this rank's "pushed" flag on every peer.
//   3. grouped GEMMs      run over the receive buffer once all sources have pushed (ep_wait); the down
//                         projection's epilogue scatters each output row into the SOURCE rank's pair
//                         buffer through the peer mapping (gemm_sm100.cu, out_peer), so the combine
//                         all-to-all is the GEMM's own store.
//   4. ep_done            flags + bounded wait: every rank's results have landed; the local combine
//                         kernel then sums each token's k rows.
// No counterpart in the reference, which mirrors tokens on every rank and sums partial outputs
// (src/model/core/tp_ep.rs:8-11).
#include "common.cuh"
#include "ep.h"

namespace lb {

__device__ __forceinline__ void ep_st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ep_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool ep_wait_geq(const uint32_t* flag, uint32_t want, uint64_t budget_ns) {
  uint64_t t0 = 0;                           // the clock (a slow read) only once the wait has lasted a while
  uint32_t spins = 0;
  while (int32_t(ep_ld_acquire(flag) - want) < 0) {
    if ((++spins & 0x3f) == 0) {
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget_ns) return false;
    }
  }
  return true;
}

// signal[slot_base + src] on rank dst is raised by rank src.
__device__ __forceinline__ void ep_signal_all(const EpPeers& p, int slot_base, uint32_t seq) {
  if (threadIdx.x < p.world) {
    __threadfence_system();
    ep_st_release(reinterpret_cast<uint32_t*>(p.signal[threadIdx.x]) + slot_base + p.rank, seq);
  }
}
__device__ __forceinline__ bool ep_wait_all(const EpPeers& p, int slot_base, uint32_t seq, uint64_t budget_ns,
                                            int* status, int* s_ok) {
  if (threadIdx.x == 0) *s_ok = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.signal[p.rank]) + slot_base + threadIdx.x;
    if (!ep_wait_geq(mine, seq, budget_ns)) {
      *s_ok = 0;
      atomicCAS(status, 0, ST_TIMEOUT_FLAG);
    }
  }
  __syncthreads();
  return *s_ok != 0;
}

// One CTA, 512 threads. counts: this rank's pairs per (global) expert.
__global__ void __launch_bounds__(512) ep_publish_counts_kernel(EpPeers p, const int* __restrict__ counts, int E,
                                                                long counts_off, const uint32_t* seq_ptr,
                                                                int* __restrict__ dest_base,
                                                                int* __restrict__ recv_counts, int* __restrict__ meta,
                                                                int cap, uint64_t budget_ns, int* status) {
  __shared__ int s_ok;
  __shared__ int s_tot[512];
  const uint32_t seq = *reinterpret_cast<const volatile uint32_t*>(seq_ptr) + 1;
  const int per = E / p.world;
  for (int r = 0; r < p.world; ++r) {
    int* tbl = reinterpret_cast<int*>(reinterpret_cast<char*>(p.buffer[r]) + counts_off) + p.rank * E;
    for (int e = threadIdx.x; e < E; e += 512) tbl[e] = counts[e];
  }
  __syncthreads();
  ep_signal_all(p, EP_SLOT_COUNTS, seq);
  if (!ep_wait_all(p, EP_SLOT_COUNTS, seq, budget_ns, status, &s_ok)) return;
  const int* all = reinterpret_cast<const int*>(reinterpret_cast<const char*>(p.buffer[p.rank]) + counts_off);
  // totals per expert over all sources
  for (int e = threadIdx.x; e < E; e += 512) {
    int t = 0;
    for (int s = 0; s < p.world; ++s) t += all[s * E + e];
    s_tot[e] = t;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += 512) {
    const int owner0 = (e / per) * per;
    int base = 0;
    for (int x = owner0; x < e; ++x) base += s_tot[x];
    for (int s = 0; s < p.rank; ++s) base += all[s * E + e];
    dest_base[e] = base;
    if (e / per == p.rank) recv_counts[e - owner0] = s_tot[e];
  }
  if (threadIdx.x == 0) {
    int rows = 0;
    for (int x = p.rank * per; x < (p.rank + 1) * per; ++x) rows += s_tot[x];
    meta[2] = rows;
    if (rows > cap) atomicCAS(status, 0, ST_BAD_ARGS);   // receive buffer too small for this routing
  }
}

// Grid-stride over this rank's sorted rows. offsets: [E + 1] local expert-major offsets of the plan.
__global__ void __launch_bounds__(128) ep_push_kernel(EpPeers p, const __nv_bfloat16* __restrict__ x, long ldx, int H,
                                                      const int* __restrict__ sorted_token,
                                                      const int* __restrict__ sorted_pair,
                                                      const float* __restrict__ sorted_w,
                                                      const int* __restrict__ offsets, const int* __restrict__ dest_base,
                                                      int E, int cap, long rx_off, long rsrc_off, long rw_off,
                                                      const uint32_t* seq_ptr, unsigned int* done_ctr) {
  const uint32_t seq = *reinterpret_cast<const volatile uint32_t*>(seq_ptr) + 1;
  const int per = E / p.world;
  const int n = offsets[E];
  for (int i = blockIdx.x; i < n; i += gridDim.x) {
    int lo = 0, hi = E;   // expert e with offsets[e] <= i < offsets[e + 1]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (offsets[mid] <= i) lo = mid; else hi = mid;
    }
    const int e = lo;
    const int d = e / per;
    const int pos = dest_base[e] + (i - offsets[e]);
    if (pos >= cap) continue;   // flagged by the count kernel
    char* base = reinterpret_cast<char*>(p.buffer[d]);
    const uint4* src = reinterpret_cast<const uint4*>(x + long(sorted_token[i]) * ldx);
    uint4* dst = reinterpret_cast<uint4*>(base + rx_off + long(pos) * H * 2);
    for (int v = threadIdx.x; v < H / 8; v += 128) dst[v] = src[v];
    if (threadIdx.x == 0) {
      reinterpret_cast<int*>(base + rsrc_off)[pos] = (p.rank << 24) | sorted_pair[i];
      reinterpret_cast<float*>(base + rw_off)[pos] = sorted_w[i];
    }
  }
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int old = atomicAdd(done_ctr, 1u);
    s_last = (old == gridDim.x - 1);
    if (s_last) *done_ctr = 0;
  }
  __syncthreads();
  if (s_last) ep_signal_all(p, EP_SLOT_PUSHED, seq);
}

// Waits for round `slot_base` of every peer; optionally raises this rank's flag first and publishes the new
// sequence number afterwards (last kernel of a layer).
__global__ void ep_sync_kernel(EpPeers p, int slot_base, int signal_first, uint32_t* seq_ptr, int bump,
                               uint64_t budget_ns, int* status) {
  __shared__ int s_ok;
  const uint32_t seq = *reinterpret_cast<const volatile uint32_t*>(seq_ptr) + 1;
  if (signal_first) ep_signal_all(p, slot_base, seq);
  ep_wait_all(p, slot_base, seq, budget_ns, status, &s_ok);
  if (bump && threadIdx.x == 0) *reinterpret_cast<volatile uint32_t*>(seq_ptr) = seq;
}

int ep_publish_counts_launch(const EpPeers& p, const int* counts, int E, long counts_off, const uint32_t* seq_ptr,
                             int* dest_base, int* recv_counts, int* meta, int cap, uint64_t budget_ns, int* status,
                             cudaStream_t s) {
  if (E > 512 || E % p.world || p.world > EP_MAX_RANKS) return 1;
  ep_publish_counts_kernel<<<1, 512, 0, s>>>(p, counts, E, counts_off, seq_ptr, dest_base, recv_counts, meta, cap,
                                             budget_ns, status);
  return cudaGetLastError() != cudaSuccess;
}

int ep_push_launch(const EpPeers& p, const void* x, long ldx, int H, const int* sorted_token, const int* sorted_pair,
                   const float* sorted_w, const int* offsets, const int* dest_base, int E, int cap, long rx_off,
                   long rsrc_off, long rw_off, const uint32_t* seq_ptr, unsigned int* done_ctr, int max_rows,
                   cudaStream_t s) {
  if (H % 8) return 1;
  int grid = max_rows < 1 ? 1 : (max_rows > 1184 ? 1184 : max_rows);
  ep_push_kernel<<<grid, 128, 0, s>>>(p, static_cast<const __nv_bfloat16*>(x), ldx, H, sorted_token, sorted_pair,
                                      sorted_w, offsets, dest_base, E, cap, rx_off, rsrc_off, rw_off, seq_ptr, done_ctr);
  return cudaGetLastError() != cudaSuccess;
}

int ep_sync_launch(const EpPeers& p, int slot_base, int signal_first, uint32_t* seq_ptr, int bump, uint64_t budget_ns,
                   int* status, cudaStream_t s) {
  ep_sync_kernel<<<1, 32, 0, s>>>(p, slot_base, signal_first, seq_ptr, bump, budget_ns, status);
  return cudaGetLastError() != cudaSuccess;
}

}  // namespace lb
