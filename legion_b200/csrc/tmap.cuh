// Host-side TMA tensor-map construction with a process-wide cache.
//
// cuTensorMapEncodeTiled is fetched through the runtime's driver entry point lookup, so the
// library links without libcuda and loads on machines that have no driver (build checks on CPU).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lb {

enum TmapDtype : int { TM_BF16 = 0, TM_U8 = 1, TM_F32 = 2 };

// 2-D row-major tensor [rows, cols] with row pitch ld_bytes; box = [box_rows, box_cols];
// swizzle128 selects CU_TENSOR_MAP_SWIZZLE_128B (box_cols * elem must then be 128 bytes).
// Returns nullptr (and sets a message retrievable with tmap_last_error) on failure.
const CUtensorMap* tmap_2d(const void* base, uint64_t rows, uint64_t cols, uint64_t ld_bytes, uint32_t box_rows,
                           uint32_t box_cols, int dtype, bool swizzle128);

// 3-D tensor [d2, d1, d0] (d0 contiguous) with byte strides s1 (between d1 steps) and s2.
const CUtensorMap* tmap_3d(const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_bytes,
                           uint64_t s2_bytes, uint32_t b0, uint32_t b1, uint32_t b2, int dtype, bool swizzle128);

const char* tmap_last_error();

}  // namespace lb
