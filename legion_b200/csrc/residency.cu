// Expert residency on the device: a decode step makes the experts it routes to resident WITHOUT a host round trip,
// so steps of an offloaded model stay inside a CUDA graph.
//
// The layer's experts live in pinned (device-mapped) host memory; n_slots of them are cached in HBM slots. The
// tables expert -> slot, slot -> expert and the decayed routing heat live in device memory. One launch per layer:
//   A. CTA 0 marks the experts of this step's routing, decays the heat, and for every routed expert that is not
//      resident picks the coldest slot whose expert this step does not use (empty slots first), records the
//      (expert, slot) pair and updates the tables;
//   B. all CTAs copy the missing experts' bytes from host memory straight into their slots (16-byte loads over
//      PCIe / C2C from the mapped host pointer: no staging copy, no stream synchronisation);
//   C. the routing is rewritten in slot numbers for the grouped GEMM.
// The CTAs of phase B wait for phase A through a flag with a deadline (status word on expiry); the grid is at most
// one CTA per SM, so all of them are resident.
//
// Counterparts in the reference: src/residency/policy.rs (decayed heat, victim choice), src/residency/staging.rs
// (copies into the slots), src/model/core/exec.rs (lookup tables in the graph).
#include "common.cuh"
#include "kernels.h"

namespace lb {
namespace {

__global__ void __launch_bounds__(1024) expert_cache_prepare_kernel(
    const int* __restrict__ ids, int n_pairs, int E, int n_slots, int* __restrict__ slot_of, int* __restrict__ expert_in,
    float* __restrict__ heat, float decay, const uint4* __restrict__ host_gu, const uint4* __restrict__ host_dn,
    uint4* __restrict__ slot_gu, uint4* __restrict__ slot_dn, long gu_vec, long dn_vec, int* __restrict__ ids_slot,
    int* __restrict__ miss_list, unsigned int* __restrict__ ctl, unsigned long long* __restrict__ stats,
    int* __restrict__ status) {
  // ctl[0]: number of misses of this launch (valid once ctl[1] == 1), ctl[1]: phase A done, ctl[2]: CTAs finished
  __shared__ unsigned char used[2048];
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ int s_miss;
  griddep_wait();
  griddep_launch();
  const int tid = threadIdx.x;
  if (blockIdx.x == 0) {
    for (int e = tid; e < E; e += blockDim.x) used[e] = 0;
    __syncthreads();
    for (int p = tid; p < n_pairs; p += blockDim.x) {
      const int e = ids[p];
      if (e >= 0 && e < E) used[e] = 1;
    }
    __syncthreads();
    for (int e = tid; e < E; e += blockDim.x) heat[e] = heat[e] * decay + (used[e] ? 1.f : 0.f);
    if (tid == 0) s_miss = 0;
    __syncthreads();
    int n_hit = 0;
    // routed experts in ascending order; one victim search (block-wide arg-min over the slots) per miss
    for (int e = 0; e < E; ++e) {
      if (!used[e]) continue;
      if (slot_of[e] >= 0) { ++n_hit; continue; }
      float best = INFINITY;
      int bs = -1;
      for (int s = tid; s < n_slots; s += blockDim.x) {
        const int x = expert_in[s];
        if (x >= 0 && used[x]) continue;                     // needed by this step
        const float h = x < 0 ? -1.f : heat[x];              // empty slots first
        if (h < best) { best = h; bs = s; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bs, o);
        if (oi >= 0 && (ov < best || (ov == best && (bs < 0 || oi < bs)))) { best = ov; bs = oi; }
      }
      if ((tid & 31) == 0) { s_val[tid >> 5] = best; s_idx[tid >> 5] = bs; }
      __syncthreads();
      if (tid == 0) {
        float b = INFINITY;
        int bi = -1;
        for (int w = 0; w < int(blockDim.x >> 5); ++w)
          if (s_idx[w] >= 0 && (s_val[w] < b || (s_val[w] == b && (bi < 0 || s_idx[w] < bi)))) { b = s_val[w]; bi = s_idx[w]; }
        if (bi < 0) {
          atomicCAS(status, 0, ST_BAD_ARGS);                 // more experts routed to than there are slots
        } else {
          const int old = expert_in[bi];
          if (old >= 0) slot_of[old] = -1;
          slot_of[e] = bi;
          expert_in[bi] = e;
          miss_list[2 * s_miss] = e;
          miss_list[2 * s_miss + 1] = bi;
          ++s_miss;
        }
      }
      __syncthreads();
    }
    if (tid == 0) {
      stats[0] += (unsigned long long)n_hit;
      stats[1] += (unsigned long long)s_miss;
      stats[2] += (unsigned long long)s_miss * (unsigned long long)(gu_vec + dn_vec) * 16ull;
      stats[3] += 1ull;
      ctl[0] = (unsigned int)s_miss;
      __threadfence();
      atomicExch(&ctl[1], 1u);
    }
  }
  // ---- phase B: every CTA waits for the plan, then copies its share of the missing experts' bytes
  __shared__ int s_ok;
  if (tid == 0) {
    s_ok = 1;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (atomicAdd(&ctl[1], 0u) == 0u) {
      if ((++spins & 0xff) == 0) {
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > 2000000000ull) {
          atomicCAS(status, 0, ST_TIMEOUT_FLAG);
          s_ok = 0;
          break;
        }
      }
    }
    __threadfence();
  }
  __syncthreads();
  if (s_ok) {
    const int n_miss = int(*reinterpret_cast<volatile unsigned int*>(&ctl[0]));
    const long per = gu_vec + dn_vec;
    const long total = long(n_miss) * per;
    for (long i = long(blockIdx.x) * blockDim.x + tid; i < total; i += long(gridDim.x) * blockDim.x) {
      const int m = int(i / per);
      const long v = i - long(m) * per;
      const int e = miss_list[2 * m], s = miss_list[2 * m + 1];
      if (v < gu_vec) slot_gu[long(s) * gu_vec + v] = host_gu[long(e) * gu_vec + v];
      else slot_dn[long(s) * dn_vec + (v - gu_vec)] = host_dn[long(e) * dn_vec + (v - gu_vec)];
    }
    // ---- phase C: routing in slot numbers
    for (long p = long(blockIdx.x) * blockDim.x + tid; p < n_pairs; p += long(gridDim.x) * blockDim.x) {
      const int e = ids[p];
      ids_slot[p] = (e >= 0 && e < E) ? __ldcg(&slot_of[e]) : -1;
    }
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const unsigned int done = atomicAdd(&ctl[2], 1u);
    if (done == gridDim.x - 1) {             // last CTA out: the control words are ready for the next launch
      ctl[0] = 0;
      ctl[1] = 0;
      ctl[2] = 0;
    }
  }
}

}  // namespace

int expert_cache_prepare_launch(const int* ids, int n_pairs, int E, int n_slots, int* slot_of, int* expert_in, float* heat,
                                float decay, const void* host_gu, const void* host_dn, void* slot_gu, void* slot_dn,
                                long gu_bytes, long dn_bytes, int* ids_slot, int* miss_list, unsigned int* ctl,
                                unsigned long long* stats, int* status, cudaStream_t s) {
  if (n_pairs <= 0) return 0;
  if (E <= 0 || E > 2048 || n_slots <= 0 || (gu_bytes % 16) || (dn_bytes % 16)) return 1;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  launch_pdl(expert_cache_prepare_kernel, dim3(sms), dim3(1024), 0, s, ids, n_pairs, E, n_slots, slot_of, expert_in, heat,
             decay, static_cast<const uint4*>(host_gu), static_cast<const uint4*>(host_dn), static_cast<uint4*>(slot_gu),
             static_cast<uint4*>(slot_dn), gu_bytes / 16, dn_bytes / 16, ids_slot, miss_list, ctl, stats, status);
  return cudaGetLastError() != cudaSuccess;
}

}  // namespace lb
