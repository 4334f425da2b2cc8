// C[M, N] = A[M, K] . W[N, K]^T (+ bias[N]) with plain 32-bit FMAs: the matrix product of the float32 path, and the
// general fallback of the bfloat16 path for sizes the tensor-core kernel refuses.
//
// Every output element is one chain of fmaf over k = 0, 1, ..., K-1 in that order, started from zero, whatever M, N,
// the tile or the thread it lands in. So a row's result has the same bits in every batch and every cutting of the
// work, and no reduced-precision mode is involved (the reference's CUDA "float32" product is a 3xTF32 tensor-core
// kernel, fusezap/device/cuda_kernels/tf32.py:1-12; its plain 32-bit product lives on its CPU device only).
//
// Tiles of 64 x 64 outputs, 16 k per stage, 256 threads with 4 x 4 outputs each; operands are converted to float32
// when staged in shared memory.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TA, typename TC>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const TA* __restrict__ W, const float* __restrict__ bias,
                 TC* __restrict__ C, int M, int N, int K) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  // staging: thread t loads row (t >> 2) and k offsets (t & 3) * 4 .. + 3 of both tiles
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  const TA* arow = A + (size_t)(m0 + lr) * K;
  const TA* wrow = W + (size_t)(n0 + lr) * K;
  const bool a_ok = m0 + lr < M, w_ok = n0 + lr < N;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      As[lk + i][lr] = (a_ok && k < K) ? Cvt<TA>::to_f(arow[k]) : 0.f;
      Ws[lk + i][lr] = (w_ok && k < K) ? Cvt<TA>::to_f(wrow[k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      C[(size_t)m * N + n] = Cvt<TC>::from_f(v);
    }
  }
}

// Few rows (M <= 16): 16 rows x 64 columns per block, 32 k per stage. A thread owns one column and four rows and walks
// k alone (splitting k over lanes would change the order of the sum); W is staged through shared memory so that the
// global reads stay coalesced.
constexpr int SM_ROWS = 16, SN = 64, SK = 32;
template <typename TA, typename TC>
__global__ void __launch_bounds__(256)
gemm_simt_small_kernel(const TA* __restrict__ A, const TA* __restrict__ W, const float* __restrict__ bias,
                       TC* __restrict__ C, int M, int N, int K) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  __shared__ float As[SK][SM_ROWS + 1];
  __shared__ float Ws[SK][SN + 1];
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * SN, m0 = blockIdx.y * SM_ROWS;
  const int tn = tid & 63, tm = tid >> 6;   // 4 row groups x 64 columns; thread does rows tm, tm+4, tm+8, tm+12
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < K; k0 += SK) {
    // W tile: 64 rows x 32 k = 2048 elements, 8 per thread; consecutive threads read consecutive k
    for (int e = tid; e < SN * SK; e += 256) {
      const int r = e >> 5, k = e & 31;
      Ws[k][r] = (n0 + r < N && k0 + k < K) ? Cvt<TA>::to_f(W[(size_t)(n0 + r) * K + k0 + k]) : 0.f;
    }
    for (int e = tid; e < SM_ROWS * SK; e += 256) {
      const int r = e >> 5, k = e & 31;
      As[k][r] = (m0 + r < M && k0 + k < K) ? Cvt<TA>::to_f(A[(size_t)(m0 + r) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SK; ++kk) {
      const float w = Ws[kk][tn];
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = fmaf(As[kk][tm + 4 * i], w, acc[i]);
    }
    __syncthreads();
  }
  const int n = n0 + tn;
  if (n < N) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int m = m0 + tm + 4 * i;
      if (m < M) {
        float v = acc[i];
        if (bias) v += bias[n];
        C[(size_t)m * N + n] = Cvt<TC>::from_f(v);
      }
    }
  }
}

template <typename TA, typename TC>
int launch(const void* A, const void* W, const float* bias, void* C, int M, int N, int K, cudaStream_t stream) {
  if (M <= SM_ROWS) {
    dim3 grid((N + SN - 1) / SN, (M + SM_ROWS - 1) / SM_ROWS);
    fz_launch(gemm_simt_small_kernel<TA, TC>, grid, dim3(256), 0, stream, (const TA*)A, (const TA*)W, bias, (TC*)C, M, N, K);
  } else {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    fz_launch(gemm_simt_kernel<TA, TC>, grid, dim3(256), 0, stream, (const TA*)A, (const TA*)W, bias, (TC*)C, M, N, K);
  }
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}
}  // namespace

// in_dtype: dtype of A and W; out_dtype: dtype of C. bias (float32) may be null.
FZ_API int fz_gemm_simt(const void* A, const void* W, const float* bias, void* C, int in_dtype, int out_dtype, int M,
                        int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return FZ_OK;
  if (K <= 0) return FZ_BAD_SHAPE;
  if ((long long)((N + 63) / 64) > 2147483647LL || (M + 15) / 16 > 65535) return FZ_TOO_LARGE;
  if (in_dtype == FZ_F32 && out_dtype == FZ_F32) return launch<float, float>(A, W, bias, C, M, N, K, stream);
  if (in_dtype == FZ_BF16 && out_dtype == FZ_F32) return launch<__nv_bfloat16, float>(A, W, bias, C, M, N, K, stream);
  if (in_dtype == FZ_BF16 && out_dtype == FZ_BF16) return launch<__nv_bfloat16, __nv_bfloat16>(A, W, bias, C, M, N, K, stream);
  return FZ_BAD_DTYPE;
}

#ifdef FZ_TIMELINE
FZ_TIMELINE_READER(gemm_simt)
#endif
