// Host interface of the weights-as-M tcgen05 GEMM (gemm_sm100.cu).
#pragma once
#include "comm.h"
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>

namespace lb {

// Device-side argument block (passed by value to the kernel).
// Optional tail of the GEMM kernel: all-reduce of the output over the ranks' symmetric buffers (+ residual, + the
// next RMSNorm). The GEMM's output must be this rank's partial slot at byte offset buf_off of its symmetric buffer.
struct WgemmCommTail {
  int enabled;
  CommPeers peers;
  long buf_off;
  int slot_base;
  uint32_t* seq_ptr;              // sequence number (device data: graph-replayable)
  unsigned int* ctrs;             // [2] arrival / exit counters, zero on entry, left zero
  int T, H;
  const __nv_bfloat16* residual; long ldr;
  __nv_bfloat16* sum_out; long lds;
  const float* norm_w; float eps, w_offset;
  __nv_bfloat16* norm_out; long ldn;
  unsigned long long budget_ns;
  int* status;                    // communicator status word
};

// Optional head of the GEMM kernel: all-gather of the activation rows. Rank r has written rows
// [r * rows_per_rank, ...) of the [T, K] activation into ITS OWN symmetric buffer at byte offset src_off (row pitch
// K elements); the kernel gathers all ranks' rows into the local tensor the X tensor map points at, then multiplies.
struct WgemmCommHead {
  int enabled;
  CommPeers peers;
  long src_off;
  int slot_base;
  uint32_t* seq_ptr;
  unsigned int* ctrs;             // [2] arrival / exit counters, zero on entry, left zero
  int T, K, rows_per_rank;
  __nv_bfloat16* x_local;         // [T, K] gather destination (= the GEMM's activation operand)
  unsigned long long budget_ns;
  int* status;
};

struct WgemmArgs {
  void* out;                      // bf16 or f32 [rows, ldo]
  long ldo;
  const __nv_bfloat16* residual;  // optional, added in the epilogue (indexed like out)
  long ldr;
  const float* tok_scale;         // optional per-activation-row multiplier
  const int* out_rows;            // optional activation-row -> output-row map (negative = drop)
  int K, n_feat, feat_tiles, n_tok;
  const int* tile_group;          // grouped mode: expert of each token tile (nullptr = dense)
  const int* tile_tok0;           //   first activation row of the tile
  const int* tile_out0;           //   first output row of the tile (nullptr = same as tile_tok0)
  const int* tile_ntok;           //   valid rows in the tile
  const int* n_tiles_dev;         //   number of token tiles (device scalar, data of a CUDA graph)
  int n_tok_tiles_max;
  int rows_per_group;             // weight rows between consecutive groups
  int x_group_col;                // grouped mode: first activation column of group g is g * x_group_col (per-head
                                  //   projections read their head's slice of a [tokens, heads * width] tensor in place)
  int dual_offset;                // DUAL: rows from a feature's gate row to its up row
  int split_k;
  int vec_ok;                     // output rows may be written as aligned 16-byte vectors
  float* ws;                      // split-K partials
  int* counters;                  // split-K arrival counters, zero on entry, left zero on exit
  int* status;                    // error word (0 = ok)
  void* out_peer[8];              // EP combine: per-rank output bases (peer-mapped); used when n_out_peer > 0,
  int n_out_peer;                 //   out_rows[] then holds (rank << 24) | row
  WgemmCommTail comm;
  WgemmCommHead head;
  const float* w_gscale;          // NVFP4 weights: per-group (x2 for DUAL: gate, up) tensor scale, applied in the epilogue
  const float* w_bscale;          // FP8 weights: fp32 scale per 128 x 128 block, [w_rows / 128, K / 128]
  const float* x_bscale;          // FP8 activations: fp32 scale per row and 128 columns, [x_rows, K / 128]
  uint8_t* q8_out;                // FP8 DUAL: the SwiGLU rows leave e4m3-encoded for the next FP8 GEMM, [rows, n_feat]
  float* q8_scale;                //   with one fp32 scale per row and 128 features, [rows, n_feat / 128]; no bf16 output
};

// Host-side description of one launch.
struct WgemmHost {
  const void* w;   long w_rows; long ldw;   // weights [w_rows, K], row pitch ldw elements
  const void* x;   long x_rows; long ldx;   // activations [x_rows, K]
  void* out; long ldo; bool out_f32;
  const __nv_bfloat16* residual; long ldr;
  const float* tok_scale;
  const int* out_rows;
  int K, n_feat, n_tok;
  int bn; bool dual;
  const int* tile_group; const int* tile_tok0; const int* tile_ntok; const int* n_tiles_dev;
  const int* tile_out0;
  int n_tok_tiles_max;
  int rows_per_group, dual_offset;
  int x_group_col; long x_cols;   // see WgemmArgs::x_group_col; x_cols: columns of the activation tensor (0 = K)
  int split_k; float* ws; int* counters;
  int* status;
  void* out_peer[8]; int n_out_peer;
  WgemmCommTail comm;
  WgemmCommHead head;
  const void* w_scales;           // non-null: w holds NVFP4 codes [rows, K/2] bytes, this the e4m3 block scales [rows, K/16]
  const float* w_gscale;
  // non-null: block-scaled FP8. w and x hold e4m3 bytes ([w_rows, K] / [x_rows, K], pitches ldw / ldx in bytes),
  // w_bscale the fp32 weight scales per 128 x 128 block, x_bscale the fp32 activation scales per row and 128 columns
  const float* w_bscale;
  const float* x_bscale;
  // FP8 DUAL only, optional: write the activated rows as e4m3 [rows, n_feat] + scales [rows, n_feat / 128] (what the
  // activation encoder would make of the bf16 rows) instead of the bf16 output
  uint8_t* q8_out;
  float* q8_scale;
};

int wgemm_launch(const WgemmHost& h, cudaStream_t stream);
int wgemm_pick_bn(int n_tok_per_tile_hint, bool dual);
size_t wgemm_workspace_floats(int bn, bool dual, int n_tok_tiles, int feat_tiles, int split_k);
const char* wgemm_last_error();

}  // namespace lb
