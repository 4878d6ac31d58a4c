// An entry point for callers that must not allocate device memory.
//
// This declaration has no counterpart in the reference project: the reference has no GPU code at
// all. It exists for programs that embed these kernels where `cudaMalloc` is off the table: a
// process whose device memory has been handed out in full to another owner (so that a further
// allocation fails or is forbidden by policy), or code that runs in a context where allocating
// CUDA calls are not permitted, such as a host function enqueued on a stream. The ordinary
// entry point, `vob_pick_tokens`, asks the caller for scratch buffers; a caller of that kind has
// nowhere to get them from. This one brings its own.
//
//   int vob_pick_tokens_static(logits, ld, R, V, temperature, seeds, steps, out, stream)
//
// picks one token per row of float32 logits [R, V] (row stride `ld` elements) exactly as
// `vob_pick_tokens` does (greedy where temperature is null or 0, Gumbel-max sampling elsewhere;
// a row that holds a NaN yields -1) and writes them to `out` (int32 [R]). All pointers are device
// pointers supplied by the caller; the partial results between its two kernels live in a fixed
// array inside the library.
//
// Limits and rules:
//   * at most VOB_PICK_STATIC_MAX_ROWS rows per call and any vocabulary size; more rows are
//     refused with VOB_ERR_STATIC_TOO_LARGE (nothing is launched);
//   * the array (VOB_PICK_STATIC_BYTES bytes) is part of the library image: every GPU that loads
//     the library holds it until the process exits;
//   * the first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current) and remembers it; make that first call outside any stream capture;
//   * every call uses the same array and finds in it whatever the last call left. The words that
//     must start at zero (the per-row NaN marks) are cleared on the stream at the start of each
//     call. (A call that ran to its end leaves them at zero itself; the clearing matters after a
//     call whose second kernel was never launched.) Two calls whose kernels may run at the same time on one GPU (different streams, no
//     ordering between them) would race on the array: order them;
//   * the function calls no cudaMalloc, cudaFree or any allocating library routine.
// Returns 0, a cudaError_t value, or one of the VOB_ERR_* codes.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define VOB_PICK_STATIC_MAX_ROWS 64
#define VOB_PICK_STATIC_MAX_SPLITS 256
// per row and split one float and one int, plus one int per row for the NaN mark
#define VOB_PICK_STATIC_BYTES (VOB_PICK_STATIC_MAX_ROWS * VOB_PICK_STATIC_MAX_SPLITS * 8 + VOB_PICK_STATIC_MAX_ROWS * 4)
#define VOB_ERR_STATIC_TOO_LARGE 2003

#ifdef __cplusplus
extern "C" {
#endif
__attribute__((visibility("default")))
int vob_pick_tokens_static(const float* logits, long long ld, int R, int V, const float* temperature,
                           const uint32_t* seeds, const int* steps, int* out, cudaStream_t stream);
// Test aid: leaves NaN marks for the first `rows` rows in the fixed array, as a call that broke off
// between its two kernels would; the next call must not be misled by them.
__attribute__((visibility("default")))
int vob_pick_static_test_leave_marks(int rows, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
