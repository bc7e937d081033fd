// Launch interface of the device-side communication kernels (comm.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define LB_MAX_RANKS 8

namespace lb {

// Peer-mapped base pointers of every rank's symmetric data buffer and signal pad (uint32 slots).
struct CommPeers {
  void* buffer[LB_MAX_RANKS];
  void* signal[LB_MAX_RANKS];
  int rank, world;
};

int wait_flag_launch(const uint32_t* flag, uint32_t want, uint64_t budget_ns, int* status, cudaStream_t s);
int barrier_launch(const CommPeers& peers, int slot_base, uint32_t seq, uint64_t budget_ns, int* status,
                   cudaStream_t s);
int all_reduce_fused_launch(const CommPeers& peers, long buf_off, int slot_base, uint32_t* seq_ptr,
                            unsigned int* done_ctr, int T, int H,
                            const void* residual, long ldr, void* sum_out, long lds, const float* norm_w, float eps,
                            float w_offset, void* norm_out, long ldn, uint64_t budget_ns, int* status,
                            cudaStream_t s);
int reduce_scatter_launch(const CommPeers& peers, long buf_off, long out_off, int slot_base, uint32_t* seq_ptr,
                          unsigned int* done_ctr, int row0, int n_rows, int H, const void* residual, long ldr, uint64_t budget_ns, int* status,
                          cudaStream_t s);
int all_gather_launch(const CommPeers& peers, long src_off, int slot_base, uint32_t* seq_ptr,
                      unsigned int* done_ctr, int T, int H, void* out,
                      long ldo, uint64_t budget_ns, int* status, cudaStream_t s);

}  // namespace lb
