// Arg-max over vocabulary rows without any allocation. This entry point has no counterpart in the
// reference engine.
//
// Who needs it: code that picks tokens from a place where device memory cannot be requested, for
// example a host callback or a plug-in running inside another framework's stream, a process whose
// memory pool has been handed over completely to the KV cache, or a C caller that links this library
// without PyTorch's allocator. The regular arg-max takes its partial-result buffers from the caller
// (PyTorch allocates them); this variant keeps them in a fixed array inside the library instead.
//
// Contract
//   * logits: device pointer, float32, `rows` rows of `vocab` values with pitch `ld` elements.
//     out: device pointer to `rows` int32 results (index of the largest value, ties to the lower index).
//   * A row that holds only NaN has no largest value: its result is 0x7fffffff (the regular arg-max
//     op answers the same), which is outside every vocabulary, so check for it if NaN rows can occur.
//     A row of -inf only answers 0.
//   * rows <= LB_NOALLOC_MAX_ROWS (256); more returns LB_NOALLOC_TOO_LARGE and launches nothing.
//   * The work is enqueued on `stream` (a cudaStream_t; 0 = default stream); nothing is synchronised.
//   * No cudaMalloc / cudaFree / allocator call is made, here or in anything it calls.
//   * The first call on each device looks up the device address of the scratch array (a few
//     microseconds of host work, with that device current); make that first call outside any stream
//     capture.
//   * All calls on one device share the 128 KiB scratch array, which keeps whatever the last call
//     left in it. Each call overwrites the part it reads, so nothing needs clearing, but two calls
//     whose kernels overlap on the GPU (different streams without ordering) race on it: order them.
#pragma once

#define LB_NOALLOC_MAX_ROWS 256
#define LB_NOALLOC_BLOCKS 64
#define LB_NOALLOC_MAX_DEVICES 64

#define LB_NOALLOC_OK 0
#define LB_NOALLOC_BAD_ARGS 1
#define LB_NOALLOC_TOO_LARGE 2
#define LB_NOALLOC_CUDA_ERROR 3

#ifdef __cplusplus
extern "C" {
#endif

int lb_argmax_noalloc(const float* logits, long ld, int rows, int vocab, int* out, void* stream);

#ifdef __cplusplus
}
#endif
