// Device helpers of the NVFP4 encoding shared by the GEMM epilogue, the activation quantiser and the reduction
// kernels that emit encoded rows: UE4M3 scale bytes, e2m1 code packing, and the byte position of a scale inside the
// 512-byte atoms that the tensor-core scale copy reads (see gemm_nvfp4_sm100.h).
#pragma once
#include <cuda_fp8.h>
#include <stdint.h>

namespace lb {

__device__ __forceinline__ float e4m3_dec(uint32_t b) {
  __nv_fp8_e4m3 v;
  v.__x = uint8_t(b);
  return float(v);
}
__device__ __forceinline__ uint32_t e4m3_enc(float f) {
  __nv_fp8_e4m3 v(f);
  return v.__x;
}
// two floats -> one byte of e2m1 codes (lo in the low nibble), round to nearest even, saturating
__device__ __forceinline__ uint32_t e2m1x2(float lo, float hi) {
  uint32_t o;
  asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u32.u8 %0, t;\n\t}" : "=r"(o) : "f"(hi), "f"(lo));
  return o;
}
__device__ __forceinline__ uint32_t pack_e2m1x8(const float (&v)[8], float inv) {
  return e2m1x2(v[0] * inv, v[1] * inv) | (e2m1x2(v[2] * inv, v[3] * inv) << 8) |
         (e2m1x2(v[4] * inv, v[5] * inv) << 16) | (e2m1x2(v[6] * inv, v[7] * inv) << 24);
}
__device__ __forceinline__ long sf_atom_byte(long row, int blk16, int k4) {
  return ((row >> 7) * k4 + (blk16 >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (blk16 & 3);
}

// Encodes 8 consecutive values of a row whose 16-element block is shared with the neighbouring lane (lane ^ 1):
// returns the 4 bytes of codes and writes the block's scale byte from the even lane. gs: the row's tensor scale.
__device__ __forceinline__ uint32_t nv4_encode8_pair(const float (&v)[8], float gs, uint8_t* sf, long row, int col8,
                                                     int k4, bool live) {
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  const uint32_t sb = e4m3_enc(amax / (6.f * gs));
  const float sdec = e4m3_dec(sb) * gs;
  const float inv = sdec > 0.f ? 1.f / sdec : 0.f;
  if (live && (col8 & 8) == 0) sf[sf_atom_byte(row, col8 >> 4, k4)] = uint8_t(sb);
  return pack_e2m1x8(v, inv);
}

}  // namespace lb
