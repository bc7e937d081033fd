// Launch interface of the Gated DeltaNet kernels (gdn.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace lb {

int conv1d_silu_launch(const void* x, long ldx, const float* w, const float* bias, float* conv_state,
                       const int* cu_seq, const int* slots, int n_seqs, int C, int KC, void* out, long ldo,
                       int write_state, cudaStream_t s, int max_len = 0);   // max_len >= 64: the token-parallel form

int gdn_recurrent_launch(const void* qkv, long ld, const float* g, const float* beta, float* state,
                         const int* cu_seq, const int* slots, int n_seqs, int Hk, int Hv, int DK, int DV,
                         int tiled_heads, float scale, float l2_eps, void* out, int write_state, int write_out,
                         int prompt_rows, cudaStream_t s);

// One launch per decode step of a Gated DeltaNet layer (conv + gates + delta rule + gated norm); see gdn.cu.
int gdn_decode_fused_launch(const void* proj, long ld, const float* conv_w, float* conv_state, int KC, const float* A,
                            const float* dt_bias, const float* norm_w, float eps, int act, float* state,
                            const int* slots, int n_seqs, int Hk, int Hv, int DK, int DV, int tiled_heads, float scale,
                            float l2_eps, void* out, cudaStream_t s);

// Chunked scan for prompt-sized steps on tensor cores (gdn_chunk_sm100.cu): 64-token chunks, heads of 128 x 128.
// blk_*: the step's 128-token blocks (first token row, valid tokens); seq_*: per sequence its first block, number of
// 64-token chunks, first token row and length. scratch: gdn_chunk_scratch_bytes(n_blocks, Hv) bytes, 256-byte aligned.
size_t gdn_chunk_scratch_bytes(int n_blocks, int Hv);
int gdn_chunk_launch(const void* qkv, long ld, long T, const float* g, const float* beta, float* state,
                     const int* blk_t0, const int* blk_n, int n_blocks, const int* seq_blk0, const int* seq_nchunk,
                     const int* seq_t0, const int* seq_len, const int* slots, int n_seqs, int Hk, int Hv, int DK, int DV,
                     int tiled_heads, float scale, float l2_eps, void* out, int write_state, void* scratch,
                     int* status, cudaStream_t s);

int gdn_gates_launch(const void* a, long lda, const void* b, long ldb, const float* A, const float* dt_bias, int Hv,
                     long T, float* g, float* beta, cudaStream_t s);

int gated_rmsnorm_launch(const void* o, const void* z, long ldz, const float* w, float eps, int DV, int Hv, long T,
                         int act, void* out, cudaStream_t s);

}  // namespace lb
