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

// Optional NVFP4 copy of the normalised rows a reduction kernel produces: codes [rows, H / 2] with pitch ld, scale
// atoms (k4 = atoms per 128 rows), one fp32 scale per row. codes == nullptr: none.
struct Nv4RowsOut {
  uint8_t* codes = nullptr;
  long ld = 0;
  uint8_t* sf = nullptr;
  float* row_gscale = nullptr;
  int k4 = 0;
};

// Optional producer of this rank's partial rows inside the decode-sized reduction: the weighted expert outputs of
// a MoE layer (one row per (token, choice) pair, rows of experts outside [e_lo, e_hi) skipped, plus one shared-expert
// row per token) are summed per token there instead of by a combine launch of their own. y == nullptr: none.
struct CombineSrc {
  const void* y = nullptr;
  long ldy = 0;
  const int* ids = nullptr;
  int k = 0, e_lo = 0, e_hi = 0;
  const void* shared = nullptr;
  long lds = 0;
};

int wait_flag_launch(const uint32_t* flag, uint32_t want, uint64_t budget_ns, int* status, cudaStream_t s);
int barrier_launch(const CommPeers& peers, int slot_base, uint32_t seq, uint64_t budget_ns, int* status,
                   cudaStream_t s);
int all_reduce_fused_launch(const CommPeers& peers, long buf_off, int slot_base, uint32_t* seq_ptr,
                            unsigned int* done_ctr, int T, int H,
                            const void* residual, long ldr, void* sum_out, long lds, const float* norm_w, float eps,
                            float w_offset, void* norm_out, long ldn, uint64_t budget_ns, int* status,
                            cudaStream_t s, const Nv4RowsOut& q = Nv4RowsOut{});
// Decode-sized one-shot all-reduce with pushed flag-carrying lines (see comm.cu). ll_off: byte offset of the staging
// areas inside every rank's symmetric buffer, 2 (alternating) x world x ll_rows x H x 4 bytes, zero before first use.
int all_reduce_ll_launch(const CommPeers& peers, long buf_off, long ll_off, int ll_rows, uint32_t* seq_ptr,
                         unsigned int* done_ctr, int T, int H, const void* residual, long ldr, void* sum_out, long lds,
                         const float* norm_w, float eps, float w_offset, void* norm_out, long ldn, uint64_t budget_ns,
                         int* status, cudaStream_t s, const Nv4RowsOut& q = Nv4RowsOut{},
                         const CombineSrc& cs = CombineSrc{});
// Greedy token of a vocabulary-split head: exchange of per-rank (best value, global token id) pairs as pushed
// flag-carrying lines; ax_off: 2 (alternating) x world x ax_rows x 16 bytes inside every rank's symmetric buffer.
int argmax_exchange_launch(const CommPeers& peers, long ax_off, int ax_rows, uint32_t* seq_ptr, unsigned int* done_ctr,
                           int rows, const float* val, const int* idx, int vocab_offset, int* picks, uint64_t budget_ns,
                           int* status, cudaStream_t s);
int reduce_scatter_launch(const CommPeers& peers, long buf_off, long out_off, int slot_base, uint32_t* seq_ptr,
                          unsigned int* done_ctr, int row0, int n_rows, int H, const void* residual, long ldr, uint64_t budget_ns, int* status,
                          cudaStream_t s, void* mc_base = nullptr);   // mc_base: NVLink multicast address of the buffers (multimem)
int all_gather_launch(const CommPeers& peers, long src_off, int slot_base, uint32_t* seq_ptr,
                      unsigned int* done_ctr, int T, int H, void* out,
                      long ldo, uint64_t budget_ns, int* status, cudaStream_t s, int local_only = 0);

}  // namespace lb
