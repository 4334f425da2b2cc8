// Shared helpers of the sm_100a kernels: dtype traits, 32-bit reductions with a fixed order, the error word.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

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
