// Host interface of the native NVFP4 (W4A4) tcgen05 GEMM (gemm_nvfp4_sm100.cu) and of the activation
// quantisers that feed it.
//
// Scale-factor layout ("atoms"). The block-scaled MMA reads its UE4M3 scale factors from tensor memory, where
// they arrive by tcgen05.cp from shared memory in chunks of 512 bytes: 32 rows of 16 bytes. One chunk (an atom)
// covers 128 matrix rows x 64 elements of K (four 16-element blocks): the scale of row r, block j sits at byte
//     (r % 32) * 16 + ((r % 128) / 32) * 4 + j
// of the atom. A scale tensor for [rows, K] is stored as [ceil(rows / 128)][k4][512] bytes with
// k4 = 4 * ceil(K / 256) atoms per row tile (K padded to whole pipeline stages, padding bytes zero), so the four
// atoms of one 256-element stage are 2048 contiguous bytes: one bulk copy.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace lb {

inline int nv4_sf_k4(long K) { return int((K + 255) / 256) * 4; }
inline size_t nv4_sf_bytes(long rows, long K) { return size_t((rows + 127) / 128) * nv4_sf_k4(K) * 512; }

struct Nv4Host {
  const uint8_t* w; long w_rows; long ldw;       // e2m1 codes [w_rows, K / 2] bytes, row pitch ldw bytes
  const uint8_t* w_sf;                            // scale atoms of the weight rows
  const float* w_gscale;                          // fp32 tensor scale per group (two per group with dual: gate, up)
  const uint8_t* x; long x_rows; long ldx;       // activation codes [x_rows, K / 2]
  const uint8_t* x_sf;                            // scale atoms of the activation rows
  const float* x_gscale; int x_gs_stride;         // fp32 scale per activation row (stride 1) or one for all (stride 0)
  void* out; long ldo;                            // bf16 [rows, ldo] (nullptr with q_codes)
  const __nv_bfloat16* residual; long ldr;
  const float* tok_scale;
  const int* out_rows;
  // quantised output instead of bf16: the epilogue result re-encoded to NVFP4 for the next GEMM
  uint8_t* q_codes; long q_ld;                    // [rows, n_feat / 2] bytes, pitch q_ld bytes
  uint8_t* q_sf;                                  // its scale atoms (k4 from n_feat)
  const float* q_gscale;                          // static fp32 tensor scale of that encoding (device scalar)
  int K, n_feat, n_tok;
  int bn; bool dual;
  // grouped mode: a tile's first activation row (tile_tok0) must be a multiple of 64 for 64-token tiles and of 128
  // for 32- and 128-token tiles (where its scale factors sit inside their 128-row atom); the kernel checks it and
  // reports ST_BAD_ARGS
  const int* tile_group; const int* tile_tok0; const int* tile_out0; const int* tile_ntok; const int* n_tiles_dev;
  int n_tok_tiles_max;
  int rows_per_group, dual_offset;
  int act;                                        // dual epilogue: 0 = SiLU, 1 = tanh-GELU
  int* status;
};

int wgemm_nv4_launch(const Nv4Host& h, cudaStream_t stream);
const char* wgemm_nv4_last_error();

// Linear scale tensor [rows, K / 16] (one UE4M3 byte per 16 elements, the checkpoint layout) -> atoms.
int nv4_pack_scales_launch(const uint8_t* scales, long rows, long K, uint8_t* atoms, cudaStream_t s);
// Atoms -> linear [rows, K / 16] (tests, de-quantisation).
int nv4_unpack_scales_launch(const uint8_t* atoms, long rows, long K, uint8_t* scales, cudaStream_t s);

// bf16 rows -> NVFP4 codes + scale atoms + fp32 row scale. Optionally fused with the residual add and RMSNorm that
// produce the rows: x (+ residual) -> sum_out; normed = rmsnorm(sum) * (w + w_offset) -> normed_out (bf16, optional)
// and its encoding. gscale_static != nullptr: every row uses that device scalar (and row_gscale is not written);
// otherwise row_gscale[r] = amax(row) / (6 * 448).
// dst row i = source row rows[i] of an encoded activation (codes, scale bytes inside their atoms, row scale), for
// i < min(*n_rows, max_rows); rows[i] < 0 skips the row. Brings token rows into the expert-sorted order of a
// routing plan without decoding them.
int nv4_gather_rows_launch(const uint8_t* codes, long ldc, const uint8_t* sf, const float* row_gscale, long K,
                           const int* rows, const int* n_rows, long max_rows, uint8_t* dst_codes, long ldd,
                           uint8_t* dst_sf, float* dst_gscale, cudaStream_t s);

int nv4_act_quant_launch(const void* x, long ldx, const void* residual, long ldr, void* sum_out, long lds,
                         const float* norm_w, float eps, float w_offset, void* normed_out, long ldn, long rows, long K,
                         const float* gscale_static, uint8_t* codes, long ldc, uint8_t* sf_atoms, float* row_gscale,
                         cudaStream_t s);

}  // namespace lb
