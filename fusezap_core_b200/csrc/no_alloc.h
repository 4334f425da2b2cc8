/* Entry point for callers that must not allocate device memory.
 *
 * This has no counterpart in the reference (fusezap/fusezap-core allocates its split-K and argmax scratch from its
 * caching allocator); it exists for host programs that cannot let a library call cudaMalloc: a program that has given
 * the whole device to a memory pool of its own, a real-time loop in which an allocation (which may synchronise the
 * device) is not acceptable, or a sandbox that forbids the allocating driver calls after start-up.
 *
 *   int fz_argmax_no_alloc(const float* logits, int* out, int rows, int vocab, cudaStream_t stream);
 *
 * Same result as fz_argmax (first index of each row's maximum; a NaN counts as the maximum and the first one wins),
 * computed by the same row-split kernel, but its scratch (partial maxima, their indices, one counter per row) lives in
 * a fixed array inside the library instead of in memory the caller allocates:
 *   - the array is FZ_NO_ALLOC_SCRATCH_BYTES (132,096 bytes) and every GPU that loads the library holds it until the
 *     process exits;
 *   - at most FZ_NO_ALLOC_MAX_ROWS (256) rows per call; a larger call is refused with FZ_TOO_LARGE (1004) and
 *     fz_no_alloc_last_error() says why; vocab has no limit;
 *   - the first call on a device looks the array's device address up (cudaGetSymbolAddress, once per device, with that
 *     device current). Make that first call outside any stream capture;
 *   - every call uses the same array, which keeps what the last call left in it. The call clears the counters it needs
 *     on `stream` before the kernel runs. Two calls that overlap on the GPU (different streams, no ordering between
 *     them) race on the array and give wrong results: order them;
 *   - the call itself allocates nothing: no cudaMalloc, cudaFree or allocating library routine.
 * Returns 0, a cudaError_t of the launch, or one of the FZ_* status codes (1001..).
 */
#pragma once
#include <cuda_runtime.h>

#define FZ_NO_ALLOC_MAX_ROWS 256
#define FZ_NO_ALLOC_MAX_SLICES 64
#define FZ_NO_ALLOC_SCRATCH_BYTES (FZ_NO_ALLOC_MAX_ROWS * FZ_NO_ALLOC_MAX_SLICES * 8 + FZ_NO_ALLOC_MAX_ROWS * 4)

#ifdef __cplusplus
extern "C" {
#endif
int fz_argmax_no_alloc(const float* logits, int* out, int rows, int vocab, cudaStream_t stream);
const char* fz_no_alloc_last_error(void);
#ifdef __cplusplus
}
#endif
