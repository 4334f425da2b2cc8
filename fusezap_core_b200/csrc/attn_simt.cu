// Paged attention with 32-bit arithmetic on CUDA cores: the attention of the float32 path (prompt portions and decoded
// tokens alike), and the general fallback of the bfloat16 path.
//
// One block per (token row, kv head, slice of up to 32 query heads of that kv head's group); warp w serves the query
// heads w, w + W, ... of the slice, so they share every key/value load. Any number of heads and any group size. Keys are walked in chunks of 32 whose boundaries are multiples of 32 in absolute
// position: chunk c holds keys 32c .. 32c+31, lane j scores key 32c+j, and the running (max, sum, accumulator) is
// updated chunk by chunk in rising c. The order of every sum therefore depends only on the row's own position and
// window, never on the batch, the cut of the prompt or the pages used (the reference's general kernel stages 32-key
// chunks in shared memory the same way: fusezap/device/cuda_kernels/attention.py:330-436).
//
//   scores s_j = (q . k_j) * scale over keys max(0, p - window + 1) <= j <= p of the row's own request (window 0: all),
//   out = sum_j exp(s_j - max) v_j / sum_j exp(s_j - max)                       (fusezap/serve/kv_cache.py:258-274)
#include "common.cuh"
#include <math.h>

namespace {
constexpr int CHUNK = 32;
constexpr int MAX_WARPS = 8;
constexpr int MAX_HPW = 4;   // query heads per warp -> up to 32 query heads per block; larger groups take more blocks
constexpr int MAX_GROUP = MAX_WARPS * MAX_HPW;
constexpr int MAX_HD = 512;

template <typename T, int DPL>   // DPL: output dims per lane = ceil(hd / 32)
__global__ void attn_simt_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                 const int* __restrict__ pos, const int* __restrict__ seq_row,
                                 const int* __restrict__ table, int mb, long long page_stride, int page_size,
                                 T* __restrict__ out, int Hq, int Hkv, int hd, float scale, int window, int* err) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  extern __shared__ float smem[];
  const int n = blockIdx.x, kvh = blockIdx.y;
  const int G_all = Hq / Hkv, g_base = blockIdx.z * MAX_GROUP;
  const int G = min(MAX_GROUP, G_all - g_base);           // the query heads of this block: g_base .. g_base + G - 1 of the group
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, W = blockDim.x >> 5;
  const int kstride = hd + 1;
  float* Ks = smem;                       // [CHUNK][hd + 1]
  float* Vs = Ks + CHUNK * kstride;       // [CHUNK][hd]
  float* Qs = Vs + CHUNK * hd;            // [G][hd]
  T* orow = out + (size_t)n * Hq * hd + ((size_t)kvh * G_all + g_base) * hd;
  const int row = seq_row[n];
  if (row < 0) {
    for (int i = threadIdx.x; i < G * hd; i += blockDim.x) orow[i] = Cvt<T>::from_f(0.f);
    return;
  }
  const int p = pos[n];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const T* qrow = q + (size_t)n * Hq * hd + ((size_t)kvh * G_all + g_base) * hd;
  for (int i = threadIdx.x; i < G * hd; i += blockDim.x) Qs[i] = Cvt<T>::to_f(qrow[i]);

  float m[MAX_HPW], l[MAX_HPW], acc[MAX_HPW][DPL];
#pragma unroll
  for (int a = 0; a < MAX_HPW; ++a) {
    m[a] = -INFINITY;
    l[a] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[a][i] = 0.f;
  }
  const int* trow = table + (size_t)row * mb;
  const long long head_off = (long long)kvh * page_size * hd;

  for (int c = lo / CHUNK; c <= p / CHUNK; ++c) {
    __syncthreads();   // the previous chunk is consumed (and Qs is written, the first time)
    for (int e = threadIdx.x; e < CHUNK * hd; e += blockDim.x) {
      const int j = e / hd, d = e - j * hd;
      const int key = c * CHUNK + j;
      float kv = 0.f, vv = 0.f;
      if (key >= lo && key <= p) {
        const int page = trow[key / page_size];
        if (page < 0) {
          atomicOr(err, FZ_ERR_NO_PAGE);
        } else {
          const long long off = (long long)page * page_stride + head_off + (long long)(key % page_size) * hd + d;
          kv = Cvt<T>::to_f(k_pool[off]);
          vv = Cvt<T>::to_f(v_pool[off]);
        }
      }
      Ks[j * kstride + d] = kv;
      Vs[j * hd + d] = vv;
    }
    __syncthreads();
    const int key = c * CHUNK + lane;
    const bool valid = key >= lo && key <= p;
#pragma unroll
    for (int a = 0; a < MAX_HPW; ++a) {
      const int g = warp + a * W;
      if (g >= G) break;
      const float* qh = Qs + g * hd;
      const float* kr = Ks + lane * kstride;
      float s = 0.f;
      for (int d = 0; d < hd; ++d) s = fmaf(qh[d], kr[d], s);
      s = valid ? s * scale : -INFINITY;
      const float mn = fmaxf(m[a], warp_max(s));       // finite: every chunk walked holds at least one visible key
      const float pj = valid ? expf(s - mn) : 0.f;
      const float corr = expf(m[a] - mn);               // 0 for the first chunk (m = -inf)
      l[a] = l[a] * corr + warp_sum(pj);
      m[a] = mn;
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[a][i] *= corr;
      for (int j = 0; j < CHUNK; ++j) {
        const float pv = __shfl_sync(0xffffffffu, pj, j);
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
          const int d = lane + 32 * i;
          if (d < hd) acc[a][i] = fmaf(pv, Vs[j * hd + d], acc[a][i]);
        }
      }
    }
  }
#pragma unroll
  for (int a = 0; a < MAX_HPW; ++a) {
    const int g = warp + a * W;
    if (g >= G) break;
    const float inv = 1.0f / l[a];
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = lane + 32 * i;
      if (d < hd) orow[g * hd + d] = Cvt<T>::from_f(acc[a][i] * inv);
    }
  }
}

template <typename T, int DPL>
int launch(const void* q, const void* k_pool, const void* v_pool, const int* pos, const int* seq_row, const int* table,
           int mb, long long page_stride, int page_size, void* out, int N, int Hq, int Hkv, int hd, float scale,
           int window, int* err, cudaStream_t stream) {
  const int G_all = Hq / Hkv, G = G_all < MAX_GROUP ? G_all : MAX_GROUP;
  const int W = G < MAX_WARPS ? G : MAX_WARPS;
  const size_t smem = sizeof(float) * ((size_t)CHUNK * (hd + 1) + (size_t)CHUNK * hd + (size_t)G * hd);
  auto kern = attn_simt_kernel<T, DPL>;
  static size_t allowed = 48 * 1024;   // per instantiation: the attribute is raised once, outside any capture
  if (smem > allowed) {
    if (smem > 227 * 1024) return FZ_TOO_LARGE;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    allowed = smem;
  }
  dim3 grid(N, Hkv, (G_all + MAX_GROUP - 1) / MAX_GROUP);
  fz_launch(kern, grid, dim3(32 * W), smem, stream, (const T*)q, (const T*)k_pool, (const T*)v_pool, pos, seq_row, table, mb,
            page_stride, page_size, (T*)out, Hq, Hkv, hd, scale, window, err);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

template <typename T>
int dispatch(const void* q, const void* k_pool, const void* v_pool, const int* pos, const int* seq_row,
             const int* table, int mb, long long page_stride, int page_size, void* out, int N, int Hq, int Hkv,
             int hd, float scale, int window, int* err, cudaStream_t stream) {
#define FZ_GO(D) return launch<T, D>(q, k_pool, v_pool, pos, seq_row, table, mb, page_stride, page_size, out, N, Hq, Hkv, hd, scale, window, err, stream)
  const int dpl = (hd + 31) / 32;
  if (dpl <= 1) FZ_GO(1);
  if (dpl <= 2) FZ_GO(2);
  if (dpl <= 4) FZ_GO(4);
  if (dpl <= 8) FZ_GO(8);
  if (dpl <= 16) FZ_GO(16);
#undef FZ_GO
  return FZ_BAD_SHAPE;
}
}  // namespace

// Sizes taken: any Hkv, Hq any multiple of Hkv, 0 < hd <= 512. Anything else returns FZ_BAD_SHAPE.
FZ_API int fz_attn_simt_check(int Hq, int Hkv, int hd) {
  if (Hq <= 0 || Hkv <= 0 || hd <= 0 || Hq % Hkv) return FZ_BAD_SHAPE;
  if (hd > MAX_HD || (Hq / Hkv + MAX_GROUP - 1) / MAX_GROUP > 65535) return FZ_BAD_SHAPE;
  return FZ_OK;
}

FZ_API int fz_attn_simt(const void* q, const void* k_pool, const void* v_pool, const int* pos, const int* seq_row,
                        const int* table, int mb, long long page_stride, int page_size, void* out, int dtype, int N,
                        int Hq, int Hkv, int hd, float scale, int window, int* err, cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (fz_attn_simt_check(Hq, Hkv, hd) != FZ_OK || page_size <= 0 || Hkv > 65535) return FZ_BAD_SHAPE;
  if (dtype == FZ_F32)
    return dispatch<float>(q, k_pool, v_pool, pos, seq_row, table, mb, page_stride, page_size, out, N, Hq, Hkv, hd, scale, window, err, stream);
  if (dtype == FZ_BF16)
    return dispatch<__nv_bfloat16>(q, k_pool, v_pool, pos, seq_row, table, mb, page_stride, page_size, out, N, Hq, Hkv, hd, scale, window, err, stream);
  return FZ_BAD_DTYPE;
}

#ifdef FZ_TIMELINE
FZ_TIMELINE_READER(attn_simt)
#endif
