// Launch interface of the block-scaled format kernels (quant.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace lb {

int nvfp4_dequant_launch(const uint8_t* codes, const uint8_t* scales, const float* global_scale, long rows, long K,
                         void* out, cudaStream_t s);
int nvfp4_quant_launch(const void* x, long ldx, const float* global_scale, long rows, long K, uint8_t* codes,
                       uint8_t* scales, cudaStream_t s);
int fp8_block_dequant_launch(const uint8_t* w, const float* scale, long rows, long K, int br, int bk, void* out,
                             cudaStream_t s);
int fp8_block_quant_launch(const void* x, long ldx, long rows, long K, int br, int bk, uint8_t* out, float* scale,
                           cudaStream_t s);
int fp8_act_quant_launch(const void* x, long ldx, long rows, long K, uint8_t* out, float* scale, cudaStream_t s);
int gguf_dequant_launch(const void* raw, int ggml_type, long n_elements, void* out_bf16, cudaStream_t s);
int randn_bf16_launch(void* out, long n, float stdv, uint64_t seed, cudaStream_t s);

}  // namespace lb
