// Shared helpers of the sm_100a kernels: dtype traits, 32-bit reductions with a fixed order, the error word.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>

#define FZ_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side
enum FzDtype : int { FZ_F32 = 0, FZ_BF16 = 1 };

// Error codes a launcher returns (0 = ok; a positive value below 1000 is a cudaError_t of the launch)
enum FzStatus : int {
  FZ_OK = 0,
  FZ_BAD_DTYPE = 1001,
  FZ_BAD_SHAPE = 1002,
  FZ_BAD_ALIGNMENT = 1003,
  FZ_TOO_LARGE = 1004,
  FZ_NO_DRIVER_ENTRY = 1005,
  FZ_TMAP_ENCODE = 1006,
};

// Bits of the device error word (kernels set them instead of faulting; the host reads and clears the word)
enum FzDeviceError : int {
  FZ_ERR_TOKEN_RANGE = 1,     // a token id outside the embedding table
  FZ_ERR_NO_PAGE = 2,         // a row's position has no page in its block table
  FZ_ERR_POS_RANGE = 4,       // a position outside the position tables
  FZ_ERR_WAIT_TIMEOUT = 8,    // a bounded wait on a barrier gave up
  FZ_ERR_ROW_RANGE = 16,      // a selected row outside the step
};

#define FZ_LAUNCH_CHECK()                          \
  do {                                             \
    cudaError_t e__ = cudaGetLastError();          \
    if (e__ != cudaSuccess) return (int)e__;       \
  } while (0)

// One rotated pair: (x1, x2) turned by the angle whose cosine and sine are c and s. Written with explicit roundings so
// that every kernel that rotates gives the same bits.
__device__ __forceinline__ void fz_rope_pair(float x1, float x2, float c, float s, float& o1, float& o2) {
  o1 = __fmaf_rn(x1, c, -__fmul_rn(x2, s));
  o2 = __fmaf_rn(x2, c, __fmul_rn(x1, s));
}

// Programmatic dependent launch. A kernel launched with `fz_launch(..., pdl = true)` may start while the kernel before
// it in the stream is still running: its blocks become resident and run their prologue early. Every kernel of this
// package therefore calls `fz_grid_wait()` before it reads or writes anything another kernel of the step touches (on
// every path, also the early-exit ones: a grid that finished without waiting would let its successor's wait return
// while an older grid still runs), and `fz_grid_launch_dependents()` to let its own successor come in early.
#ifndef FZ_TIMELINE
__device__ __forceinline__ void fz_grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void fz_grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#else
// Measurement aid (a library built with -DFZ_TIMELINE): thread 0 of block (0, 0, 0) of every launch notes the global
// timer when the block starts and when its wait on the kernels before returns, two numbers per launch in launch order,
// in a buffer of the source file the kernel is compiled in (`fz_timeline_<file>` reads and clears it). The difference of
// two successive launches' second numbers is what the earlier kernel costs on the step's critical path; the first
// number says how early a kernel's blocks were resident.
static __device__ unsigned long long fz_tl_buf[2 * 4096];
static __device__ unsigned int fz_tl_n;
__device__ __forceinline__ unsigned long long fz_tl_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool fz_tl_me() { return (blockIdx.x | blockIdx.y | blockIdx.z | threadIdx.x | threadIdx.y) == 0; }
__device__ __forceinline__ unsigned int& fz_tl_slot() {
  __shared__ unsigned int slot;
  return slot;
}
__device__ __forceinline__ void fz_grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (fz_tl_me()) {
    const unsigned int s = atomicAdd(&fz_tl_n, 1u);
    fz_tl_slot() = s;
    if (s < 4096u) { fz_tl_buf[2 * s] = fz_tl_now(); fz_tl_buf[2 * s + 1] = 0; }
  }
}
__device__ __forceinline__ void fz_grid_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (fz_tl_me()) {
    const unsigned int s = fz_tl_slot();
    if (s < 4096u && fz_tl_buf[2 * s + 1] == 0) fz_tl_buf[2 * s + 1] = fz_tl_now();
  }
}
#define FZ_TIMELINE_READER(name)                                                                          \
  extern "C" __attribute__((visibility("default"))) int fz_timeline_##name(unsigned long long* host, unsigned int* n) { \
    cudaError_t e = cudaMemcpyFromSymbol(n, fz_tl_n, sizeof(unsigned int));                               \
    if (e == cudaSuccess) e = cudaMemcpyFromSymbol(host, fz_tl_buf, sizeof(fz_tl_buf));                   \
    const unsigned int zero = 0;                                                                          \
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(fz_tl_n, &zero, sizeof(unsigned int));                   \
    return (int)e;                                                                                        \
  }
#endif

// FZB200_PDL=0 in the environment turns programmatic dependent launch off (plain stream order).
inline bool fz_pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("FZB200_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t fz_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = fz_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename T> struct Cvt;
template <> struct Cvt<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds 32 floats. The order of the
// additions depends only on the block size, so a row's sum never depends on the rest of the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < nwarp ? scratch[lane] : 0.f;
  r = warp_sum(r);
  return r;
}
