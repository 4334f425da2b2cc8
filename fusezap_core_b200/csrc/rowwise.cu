// Row kernels of the step: embedding gather, residual add + RMSNorm, rotation + paged cache write, SwiGLU, argmax,
// temperature sampling. One block per token row (or a grid-stride loop for the elementwise one). Every reduction is in
// 32-bit with an order fixed by the row length and the block size only.
//
// What each computes follows the reference's serve kernels (fusezap/serve/cuda.py:161-258 RMSNorm, :284-315 SwiGLU,
// :317-427 rotation with cache write, :431-479 argmax, :547-575 step inputs); the residual stream is kept in float32
// here, so the norm rounds once where the reference rounds x + d, y and w*y separately.
#include "common.cuh"
#include <math.h>

// ------------------------------------------------------------------------------------------------ embedding
// src (may be null): src[n] >= 0 takes the row's token from prev_ids[src[n]] (the ids the previous step chose, still on
// the device) instead of tokens[n]. scale: every value is multiplied by it in float32 (1 for the models that do not
// scale their embeddings: the product is then exact).
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens, const int* __restrict__ src,
                             const int* __restrict__ prev_ids, float* __restrict__ x, int D, int V, float scale, int* err) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  const int n = blockIdx.x;
  int tok = tokens[n];
  if (src != nullptr && src[n] >= 0) tok = prev_ids[src[n]];
  float* xr = x + (size_t)n * D;
  if (tok < 0 || tok >= V) {
    if (threadIdx.x == 0) atomicOr(err, FZ_ERR_TOKEN_RANGE);
    for (int d = threadIdx.x; d < D; d += blockDim.x) xr[d] = 0.f;
    return;
  }
  const T* tr = table + (size_t)tok * D;
  if (D % 8 == 0 && ((((uintptr_t)tr) | ((uintptr_t)xr)) & 15) == 0) {
    // 16 bytes of the table row per thread and turn (8 bf16 or 4 float32 values): one round of loads for a row of 4096
    constexpr int PER = 16 / (int)sizeof(T);
    for (int d = threadIdx.x * PER; d < D; d += blockDim.x * PER) {
      const uint4 raw = *(const uint4*)(tr + d);
      const T* v = (const T*)&raw;
      float f[PER];
#pragma unroll
      for (int i = 0; i < PER; ++i) f[i] = __fmul_rn(Cvt<T>::to_f(v[i]), scale);
#pragma unroll
      for (int i = 0; i < PER; i += 4) *(float4*)(xr + d + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
    }
    return;
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) xr[d] = __fmul_rn(Cvt<T>::to_f(tr[d]), scale);
}

FZ_API int fz_embed(const void* table, int table_dtype, const int* tokens, const int* src, const int* prev_ids, float* x,
                    int N, int D, int V, float scale, int* err, cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (table_dtype == FZ_F32)
    fz_launch(embed_kernel<float>, dim3(N), dim3(512), 0, stream, (const float*)table, tokens, src, prev_ids, x, D, V, scale, err);
  else if (table_dtype == FZ_BF16)
    fz_launch(embed_kernel<__nv_bfloat16>, dim3(N), dim3(512), 0, stream, (const __nv_bfloat16*)table, tokens, src, prev_ids, x, D, V, scale, err);
  else
    return FZ_BAD_DTYPE;
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

// ------------------------------------------------------------------------------------------------ add + RMSNorm
// rows == nullptr: x[n] += delta[n] (in place), h[n] = w * x[n] * rsqrt(mean(x[n]^2) + eps), one block per row n.
// rows != nullptr: block r reads row rows[r] (x + delta, x untouched) and writes h[r]; rows[r] < 0 gives zeros.
template <typename TW, typename TH>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta, const TW* __restrict__ w,
                                   TH* __restrict__ h, const int* __restrict__ rows, int n_src, int D, float eps,
                                   int* err) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  int src = r;
  TH* hr = h + (size_t)r * D;
  if (rows != nullptr) {
    src = rows[r];
    if (src < 0 || src >= n_src) {
      if (src >= n_src && threadIdx.x == 0) atomicOr(err, FZ_ERR_ROW_RANGE);
      for (int d = threadIdx.x; d < D; d += blockDim.x) hr[d] = Cvt<TH>::from_f(0.f);
      return;
    }
  }
  float* xr = x + (size_t)src * D;
  const float* dr = delta ? delta + (size_t)src * D : nullptr;
  const bool write_x = rows == nullptr && dr != nullptr;
  float ss = 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v = xr[d];
    if (dr) v += dr[d];
    if (write_x) xr[d] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss * (1.0f / (float)D) + eps);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v = xr[d];
    if (dr && !write_x) v += dr[d];
    hr[d] = Cvt<TH>::from_f(Cvt<TW>::to_f(w[d]) * (v * scale));
  }
}

// The same for D % 4 == 0 and D <= 4 * 512 * VPT: 512 threads, a thread keeps its VPT float4 groups of the row in
// registers (all loads are issued before anything depends on them), so the row is read once.
__device__ __forceinline__ float4 load4f(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ float4 load4f(const __nv_bfloat16* p) {
  const uint2 u = *(const uint2*)p;
  const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&u.x), b = __bfloat1622float2(*(const __nv_bfloat162*)&u.y);
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4f(float* d, float a, float b, float c, float e) { *(float4*)d = make_float4(a, b, c, e); }
__device__ __forceinline__ void store4f(__nv_bfloat16* d, float a, float b, float c, float e) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, e);
  *(uint2*)d = make_uint2(*(const uint32_t*)&lo, *(const uint32_t*)&hi);
}

template <typename TW, typename TH, int VPT, bool EARLY>
__global__ void __launch_bounds__(512)
add_rmsnorm_vec_kernel(float* __restrict__ x, const float* __restrict__ delta, const TW* __restrict__ w,
                       TH* __restrict__ h, const int* __restrict__ rows, int n_src, int D, float eps, int* err) {
  fz_grid_launch_dependents();
  const int r = blockIdx.x;
  const int D4 = D >> 2;
  // EARLY (w and h 16-byte aligned): the norm's weights, and which row the block reads, depend on nothing a kernel before
  // this one writes (weights; the step's metadata, packed by the host before the step's first kernel), so they are
  // asked for ahead of the wait on that kernel instead of after the reduction. Two engines alternating in one process,
  // Llama-3.1-8B sizes: a batch-1 decode step 3.175 -> 3.128 ms, batch 8 and 64 unchanged.
  float4 g[VPT];
  int src = r;
  if constexpr (EARLY) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * 512;
      g[i] = c < D4 ? load4f(w + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (rows != nullptr) src = rows[r];
  }
  fz_grid_wait();
  __shared__ float scratch[32];
  TH* hr = h + (size_t)r * D;
  if (rows != nullptr) {
    if constexpr (!EARLY) src = rows[r];
    if (src < 0 || src >= n_src) {
      if (src >= n_src && threadIdx.x == 0) atomicOr(err, FZ_ERR_ROW_RANGE);
      for (int d = threadIdx.x; d < D; d += blockDim.x) hr[d] = Cvt<TH>::from_f(0.f);
      return;
    }
  }
  float4* xr = (float4*)(x + (size_t)src * D);
  const float4* dr = delta ? (const float4*)(delta + (size_t)src * D) : nullptr;
  const bool write_x = rows == nullptr && dr != nullptr;
  float4 v[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * 512;
    v[i] = c < D4 ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (dr) {
    float4 dv[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * 512;
      dv[i] = c < D4 ? dr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) { v[i].x += dv[i].x; v[i].y += dv[i].y; v[i].z += dv[i].z; v[i].w += dv[i].w; }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss); ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
  }
  if (write_x) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * 512;
      if (c < D4) xr[c] = v[i];
    }
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss * (1.0f / (float)D) + eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * 512;
    if (c < D4) {
      const int d = c * 4;
      if constexpr (EARLY) {
        store4f(hr + d, g[i].x * (v[i].x * scale), g[i].y * (v[i].y * scale), g[i].z * (v[i].z * scale), g[i].w * (v[i].w * scale));
        continue;
      }
      hr[d] = Cvt<TH>::from_f(Cvt<TW>::to_f(w[d]) * (v[i].x * scale));
      hr[d + 1] = Cvt<TH>::from_f(Cvt<TW>::to_f(w[d + 1]) * (v[i].y * scale));
      hr[d + 2] = Cvt<TH>::from_f(Cvt<TW>::to_f(w[d + 2]) * (v[i].z * scale));
      hr[d + 3] = Cvt<TH>::from_f(Cvt<TW>::to_f(w[d + 3]) * (v[i].w * scale));
    }
  }
}

template <typename TW, typename TH>
static int launch_norm(float* x, const float* delta, const void* w, void* h, const int* rows, int n_out, int n_src, int D,
                       float eps, int* err, cudaStream_t stream) {
  const bool vec = D % 4 == 0 && D <= 4 * 512 * 8 && (((uintptr_t)x | (uintptr_t)delta) & 15) == 0;
  const bool early = (((uintptr_t)w | (uintptr_t)h) & 15) == 0;      // vector loads of the weights, vector stores of h
  if (vec) {
    const int groups = (D / 4 + 511) / 512;
#define FZ_V(V) do { if (early) fz_launch(add_rmsnorm_vec_kernel<TW, TH, V, true>, dim3(n_out), dim3(512), 0, stream, x, delta, (const TW*)w, (TH*)h, rows, n_src, D, eps, err); \
    else fz_launch(add_rmsnorm_vec_kernel<TW, TH, V, false>, dim3(n_out), dim3(512), 0, stream, x, delta, (const TW*)w, (TH*)h, rows, n_src, D, eps, err); } while (0)
    if (groups <= 1) FZ_V(1); else if (groups <= 2) FZ_V(2); else if (groups <= 4) FZ_V(4); else FZ_V(8);
#undef FZ_V
  } else {
    fz_launch(add_rmsnorm_kernel<TW, TH>, dim3(n_out), dim3(256), 0, stream, x, delta, (const TW*)w, (TH*)h, rows, n_src, D, eps, err);
  }
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_add_rmsnorm(float* x, const float* delta, const void* w, int w_dtype, void* h, int h_dtype,
                          const int* rows, int n_out, int n_src, int D, float eps, int* err, cudaStream_t stream) {
  if (n_out <= 0) return FZ_OK;
#define FZ_NORM(TW, TH) return launch_norm<TW, TH>(x, delta, w, h, rows, n_out, n_src, D, eps, err, stream)
  if (w_dtype == FZ_F32 && h_dtype == FZ_F32) FZ_NORM(float, float);
  if (w_dtype == FZ_F32 && h_dtype == FZ_BF16) FZ_NORM(float, __nv_bfloat16);
  if (w_dtype == FZ_BF16 && h_dtype == FZ_BF16) FZ_NORM(__nv_bfloat16, __nv_bfloat16);
  if (w_dtype == FZ_BF16 && h_dtype == FZ_F32) FZ_NORM(__nv_bfloat16, float);
#undef FZ_NORM
  return FZ_BAD_DTYPE;
}

// ------------------------------------------------------------------------------------------------ rotation + cache write
// qkv: (N, (Hq + 2 Hkv) * hd) float32. One block per row. Pair (j, j + hd/2) of every q and k head is rotated by the
// angle of the row's position; q goes to q_out, k and v to the row's slot of the paged pool.
template <typename T>
__global__ void rope_kv_write_kernel(const float* __restrict__ qkv, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, const int* __restrict__ pos,
                                     const int* __restrict__ seq_row, const int* __restrict__ table, int mb,
                                     T* __restrict__ k_pool, T* __restrict__ v_pool, long long page_stride,
                                     int page_size, int write, T* __restrict__ q_out, int Hq, int Hkv, int hd,
                                     int max_len, int* err) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  const int n = blockIdx.x;
  const int half = hd >> 1;
  const int row = seq_row[n];
  T* qo = q_out + (size_t)n * Hq * hd;
  if (row < 0) {
    for (int i = threadIdx.x; i < Hq * hd; i += blockDim.x) qo[i] = Cvt<T>::from_f(0.f);
    return;
  }
  const int p = pos[n];
  if (p < 0 || p >= max_len) {
    if (threadIdx.x == 0) atomicOr(err, FZ_ERR_POS_RANGE);
    for (int i = threadIdx.x; i < Hq * hd; i += blockDim.x) qo[i] = Cvt<T>::from_f(0.f);
    return;
  }
  const float* in = qkv + (size_t)n * (Hq + 2 * Hkv) * hd;
  const float* cr = cos_t + (size_t)p * half;
  const float* sr = sin_t + (size_t)p * half;
  long long slot_base = -1;
  if (write) {
    const int page = table[(size_t)row * mb + p / page_size];
    if (page < 0) {
      if (threadIdx.x == 0) atomicOr(err, FZ_ERR_NO_PAGE);
    } else {
      slot_base = (long long)page * page_stride + (long long)(p % page_size) * hd;
    }
  }
  const long long head_stride = (long long)page_size * hd;
  // rotated pairs of the q and k heads
  for (int i = threadIdx.x; i < (Hq + Hkv) * half; i += blockDim.x) {
    const int head = i / half, j = i - head * half;
    const float x1 = in[head * hd + j], x2 = in[head * hd + j + half];
    float o1, o2;
    fz_rope_pair(x1, x2, cr[j], sr[j], o1, o2);
    if (head < Hq) {
      qo[head * hd + j] = Cvt<T>::from_f(o1);
      qo[head * hd + j + half] = Cvt<T>::from_f(o2);
    } else if (slot_base >= 0) {
      T* kd = k_pool + slot_base + (long long)(head - Hq) * head_stride;
      kd[j] = Cvt<T>::from_f(o1);
      kd[j + half] = Cvt<T>::from_f(o2);
    }
  }
  if (slot_base >= 0) {
    const float* vin = in + (Hq + Hkv) * hd;
    for (int i = threadIdx.x; i < Hkv * hd; i += blockDim.x) {
      const int head = i / hd, j = i - head * hd;
      v_pool[slot_base + (long long)head * head_stride + j] = Cvt<T>::from_f(vin[i]);
    }
  }
}

// The same for head sizes that are multiples of 8: grid (rows, blocks of heads); a thread owns four neighbouring pairs of
// one head (float4 loads, one vector store per half), so a decode step's few rows still spread over many blocks. The
// row's metadata and angles do not depend on the kernel before and are read ahead of the wait on it.
__device__ __forceinline__ void store4(float* d, float a, float b, float c, float e) { *(float4*)d = make_float4(a, b, c, e); }
__device__ __forceinline__ void store4(__nv_bfloat16* d, float a, float b, float c, float e) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, e);
  *(uint2*)d = make_uint2(*(const uint32_t*)&lo, *(const uint32_t*)&hi);
}

template <typename T>
__global__ void rope_kv_write_vec_kernel(const float* __restrict__ qkv, const float* __restrict__ cos_t,
                                         const float* __restrict__ sin_t, const int* __restrict__ pos,
                                         const int* __restrict__ seq_row, const int* __restrict__ table, int mb,
                                         T* __restrict__ k_pool, T* __restrict__ v_pool, long long page_stride,
                                         int page_size, int write, T* __restrict__ q_out, int Hq, int Hkv, int hd,
                                         int max_len, int* err) {
  fz_grid_launch_dependents();
  const int n = blockIdx.x;
  const int half = hd >> 1, per_head = half >> 2;
  const int item = blockIdx.y * blockDim.x + threadIdx.x;
  const int head = item / per_head, j = (item - head * per_head) * 4;
  const bool active = head < Hq + 2 * Hkv;
  const int row = seq_row[n];
  const int p = pos[n];
  const bool in_range = p >= 0 && p < max_len;
  float4 c = make_float4(1.f, 1.f, 1.f, 1.f), sn = make_float4(0.f, 0.f, 0.f, 0.f);
  long long slot_base = -1;
  bool no_page = false;
  if (active && row >= 0 && in_range) {
    if (head < Hq + Hkv) {
      c = *(const float4*)(cos_t + (size_t)p * half + j);
      sn = *(const float4*)(sin_t + (size_t)p * half + j);
    }
    if (write && head >= Hq) {
      const int page = table[(size_t)row * mb + p / page_size];
      no_page = page < 0;
      if (!no_page) slot_base = (long long)page * page_stride + (long long)(p % page_size) * hd;
    }
  }
  fz_grid_wait();
  if (!active) return;
  if (row < 0 || !in_range) {
    if (row >= 0 && item == 0) atomicOr(err, FZ_ERR_POS_RANGE);
    if (head < Hq) {
      T* qo = q_out + ((size_t)n * Hq + head) * hd;
      store4(qo + j, 0.f, 0.f, 0.f, 0.f);
      store4(qo + j + half, 0.f, 0.f, 0.f, 0.f);
    }
    return;
  }
  if (no_page && j == 0 && head == Hq) atomicOr(err, FZ_ERR_NO_PAGE);
  const float* in = qkv + ((size_t)n * (Hq + 2 * Hkv) + head) * hd;
  const float4 x1 = *(const float4*)(in + j), x2 = *(const float4*)(in + j + half);
  // (for the value heads c = 1 and sn = 0: the values pass unchanged)
  float a0, a1, a2, a3, b0, b1, b2, b3;
  fz_rope_pair(x1.x, x2.x, c.x, sn.x, a0, b0);
  fz_rope_pair(x1.y, x2.y, c.y, sn.y, a1, b1);
  fz_rope_pair(x1.z, x2.z, c.z, sn.z, a2, b2);
  fz_rope_pair(x1.w, x2.w, c.w, sn.w, a3, b3);
  T* dst;
  if (head < Hq) {
    dst = q_out + ((size_t)n * Hq + head) * hd;
  } else {
    if (slot_base < 0) return;
    const long long head_stride = (long long)page_size * hd;
    dst = head < Hq + Hkv ? k_pool + slot_base + (long long)(head - Hq) * head_stride
                          : v_pool + slot_base + (long long)(head - Hq - Hkv) * head_stride;
  }
  if (head < Hq + Hkv) {
    store4(dst + j, a0, a1, a2, a3);
    store4(dst + j + half, b0, b1, b2, b3);
  } else {
    store4(dst + j, x1.x, x1.y, x1.z, x1.w);
    store4(dst + j + half, x2.x, x2.y, x2.z, x2.w);
  }
}

FZ_API int fz_rope_kv_write(const float* qkv, const float* cos_t, const float* sin_t, const int* pos,
                            const int* seq_row, const int* table, int mb, void* k_pool, void* v_pool,
                            long long page_stride, int page_size, int write, void* q_out, int dtype, int N, int Hq,
                            int Hkv, int hd, int max_len, int* err, cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (hd % 2 || hd <= 0) return FZ_BAD_SHAPE;
  if (dtype != FZ_F32 && dtype != FZ_BF16) return FZ_BAD_DTYPE;
  const bool aligned = ((((uintptr_t)qkv | (uintptr_t)cos_t | (uintptr_t)sin_t | (uintptr_t)k_pool | (uintptr_t)v_pool |
                          (uintptr_t)q_out) & 15) == 0) && page_stride % 8 == 0;
  if (hd % 8 == 0 && aligned) {
    const int items = (Hq + 2 * Hkv) * (hd / 8);
    const int threads = items < 256 ? ((items + 31) / 32) * 32 : 256;
    dim3 grid(N, (items + threads - 1) / threads);
    if (dtype == FZ_F32)
      fz_launch(rope_kv_write_vec_kernel<float>, grid, dim3(threads), 0, stream, qkv, cos_t, sin_t, pos, seq_row, table, mb,
                (float*)k_pool, (float*)v_pool, page_stride, page_size, write, (float*)q_out, Hq, Hkv, hd, max_len, err);
    else
      fz_launch(rope_kv_write_vec_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, qkv, cos_t, sin_t, pos, seq_row,
                table, mb, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, page_stride, page_size, write,
                (__nv_bfloat16*)q_out, Hq, Hkv, hd, max_len, err);
    FZ_LAUNCH_CHECK();
    return FZ_OK;
  }
  if (dtype == FZ_F32)
    fz_launch(rope_kv_write_kernel<float>, dim3(N), dim3(256), 0, stream, qkv, cos_t, sin_t, pos, seq_row, table, mb,
              (float*)k_pool, (float*)v_pool, page_stride, page_size, write, (float*)q_out, Hq, Hkv, hd, max_len, err);
  else if (dtype == FZ_BF16)
    fz_launch(rope_kv_write_kernel<__nv_bfloat16>, dim3(N), dim3(256), 0, stream, qkv, cos_t, sin_t, pos, seq_row, table,
              mb, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, page_stride, page_size, write, (__nv_bfloat16*)q_out,
              Hq, Hkv, hd, max_len, err);
  else
    return FZ_BAD_DTYPE;
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

// ------------------------------------------------------------------------------------------------ SwiGLU
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, long long total, int I) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long n = idx / I;
    const int i = (int)(idx - n * I);
    const float g = Cvt<T>::to_f(gu[n * 2 * I + i]);
    const float u = Cvt<T>::to_f(gu[n * 2 * I + I + i]);
    out[idx] = Cvt<T>::from_f(g / (1.0f + expf(-g)) * u);
  }
}

// 16 bytes of gate and of up per thread (8 bf16 or 4 float32); needs I a multiple of that count and aligned operands.
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, long long groups, int I) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  constexpr int V = 16 / sizeof(T);
  const int per_row = I / V;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < groups;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long n = idx / per_row;
    const int i = (int)(idx - n * per_row) * V;
    const uint4 gq = *(const uint4*)(gu + n * 2 * I + i);
    const uint4 uq = *(const uint4*)(gu + n * 2 * I + I + i);
    const T* g = (const T*)&gq;
    const T* u = (const T*)&uq;
    uint4 oq;
    T* o = (T*)&oq;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float gf = Cvt<T>::to_f(g[j]);
      o[j] = Cvt<T>::from_f(gf / (1.0f + expf(-gf)) * Cvt<T>::to_f(u[j]));
    }
    *(uint4*)(out + n * I + i) = oq;
  }
}

template <typename T>
static int launch_swiglu(const void* gu, void* out, int N, int I, cudaStream_t stream) {
  constexpr int V = 16 / sizeof(T);
  const long long total = (long long)N * I;
  const int block = 256;
  if (I % V == 0 && ((((uintptr_t)gu) | ((uintptr_t)out)) & 15) == 0) {
    const long long groups = total / V;
    long long blocks = (groups + block - 1) / block;
    if (blocks > 148LL * 16) blocks = 148LL * 16;
    fz_launch(swiglu_vec_kernel<T>, dim3((int)blocks), dim3(block), 0, stream, (const T*)gu, (T*)out, groups, I);
  } else {
    long long blocks = (total + block - 1) / block;
    if (blocks > 148LL * 32) blocks = 148LL * 32;
    fz_launch(swiglu_kernel<T>, dim3((int)blocks), dim3(block), 0, stream, (const T*)gu, (T*)out, total, I);
  }
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_swiglu(const void* gu, void* out, int dtype, int N, int I, cudaStream_t stream) {
  if ((long long)N * I <= 0) return FZ_OK;
  if (dtype == FZ_F32) return launch_swiglu<float>(gu, out, N, I, stream);
  if (dtype == FZ_BF16) return launch_swiglu<__nv_bfloat16>(gu, out, N, I, stream);
  return FZ_BAD_DTYPE;
}

// ------------------------------------------------------------------------------------------------ argmax / sampling
// (value, index) order of numpy.argmax: a NaN is the maximum, among equals the lower index wins.
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
  const bool vn = isnan(v), bn = isnan(bv);
  if (vn != bn) return vn;
  if (vn) return i < bi;
  if (v != bv) return v > bv;
  return i < bi;
}

__device__ int block_argmax(const float* __restrict__ row, int V, float* s_val, int* s_idx) {
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (bi == 0x7fffffff || better(v, i, bv, bi)) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (oi != 0x7fffffff && (bi == 0x7fffffff || better(ov, oi, bv, bi))) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) { s_val[warp] = bv; s_idx[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = lane < nwarp ? s_val[lane] : -INFINITY;
    bi = lane < nwarp ? s_idx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || better(ov, oi, bv, bi))) { bv = ov; bi = oi; }
    }
    if (lane == 0) s_idx[0] = bi;
  }
  __syncthreads();
  const int res = s_idx[0];
  __syncthreads();
  return res;
}

// Argmax of a row split over `gridDim.y` CTAs: each takes a contiguous slice and leaves its (value, index) in
// `partial`; the CTA that arrives last at the row's counter reduces the slices in index order and resets the counter.
__global__ void argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int V, float* partial_val,
                              int* partial_idx, int* counters) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ int s_last;
  const int r = blockIdx.x, S = gridDim.y, c = blockIdx.y;
  const int chunk = (V + S - 1) / S;
  const int lo = min(V, c * chunk), hi = min(V, lo + chunk);
  const float* row = logits + (size_t)r * V;
  int res = block_argmax(row + lo, hi - lo, s_val, s_idx);
  if (threadIdx.x == 0) {
    const bool empty = hi <= lo;
    partial_val[r * S + c] = empty ? -INFINITY : row[lo + res];
    partial_idx[r * S + c] = empty ? 0x7fffffff : lo + res;
    __threadfence();
    const int old = atomicAdd(&counters[r], 1);
    s_last = old == S - 1;
    if (s_last) counters[r] = 0;
  }
  __syncthreads();
  if (!s_last || threadIdx.x != 0) return;
  __threadfence();
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = 0; i < S; ++i) {
    const float v = __ldcg(&partial_val[r * S + i]);
    const int ix = __ldcg(&partial_idx[r * S + i]);
    if (ix != 0x7fffffff && (bi == 0x7fffffff || better(v, ix, bv, bi))) { bv = v; bi = ix; }
  }
  out[r] = bi == 0x7fffffff ? 0 : bi;
}

// scratch: float partial_val[R * S], int partial_idx[R * S], int counters[R] (zero before the first call; the kernel
// leaves them zero). S = fz_argmax_slices(V).
constexpr int FZ_ARGMAX_MAX_SLICES = 64;
FZ_API int fz_argmax_max_slices(void) { return FZ_ARGMAX_MAX_SLICES; }
FZ_API int fz_argmax_slices(int V) {
  const int s = (V + 8191) / 8192;
  return s < 1 ? 1 : (s > FZ_ARGMAX_MAX_SLICES ? FZ_ARGMAX_MAX_SLICES : s);
}

FZ_API int fz_argmax(const float* logits, int* out, int R, int V, float* partial_val, int* partial_idx, int* counters,
                     cudaStream_t stream) {
  if (R <= 0) return FZ_OK;
  if (V <= 0) return FZ_BAD_SHAPE;
  dim3 grid(R, fz_argmax_slices(V));
  fz_launch(argmax_kernel, grid, dim3(512), 0, stream, logits, out, V, partial_val, partial_idx, counters);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

// out[r]: first index whose running sum of exp((l - max) / T) in float64, taken in index order, exceeds u * total.
// Thread t owns the contiguous range [t * chunk, (t + 1) * chunk), so partial sums are in index order.
__global__ void sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                              const double* __restrict__ uniform, int* __restrict__ out, int V) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ double s_sum[1024];
  __shared__ double s_target;
  __shared__ int s_res;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * V;
  const float T = temperature[r];
  const int amax = block_argmax(row, V, s_val, s_idx);
  if (!(T > 0.f)) {
    if (threadIdx.x == 0) out[r] = amax;
    return;
  }
  const double mx = (double)row[amax] / (double)T;
  const int chunk = (V + blockDim.x - 1) / blockDim.x;
  const int lo = min(V, (int)threadIdx.x * chunk), hi = min(V, lo + chunk);
  double local = 0.0;
  for (int i = lo; i < hi; ++i) local += exp((double)row[i] / (double)T - mx);
  s_sum[threadIdx.x] = local;
  __syncthreads();
  if (threadIdx.x == 0) {   // exclusive prefix over the threads' ranges, in index order
    double run = 0.0;
    for (int t = 0; t < (int)blockDim.x; ++t) {
      const double v = s_sum[t];
      s_sum[t] = run;
      run += v;
    }
    s_target = uniform[r] * run;
    s_res = V - 1;
  }
  __syncthreads();
  const double target = s_target;
  const double excl = s_sum[threadIdx.x];
  if (lo < hi && excl <= target && excl + local > target) {
    double run = excl;
    int res = hi - 1;
    for (int i = lo; i < hi; ++i) {
      run += exp((double)row[i] / (double)T - mx);
      if (run > target) { res = i; break; }
    }
    s_res = res;
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = s_res;
}

FZ_API int fz_sample(const float* logits, const float* temperature, const double* uniform, int* out, int R, int V,
                     cudaStream_t stream) {
  if (R <= 0) return FZ_OK;
  if (V <= 0) return FZ_BAD_SHAPE;
  fz_launch(sample_kernel, dim3(R), dim3(1024), 0, stream, logits, temperature, uniform, out, V);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

// ------------------------------------------------------------------------------------------------ top-k / top-p sampling
// The reference's host sampler on the device (fusezap/serve/sampling.py:25-45, 61-73): logits / T in float64; top-k keeps
// everything not below the k-th largest value (ties stay); top-p keeps, in falling order of value (ties by rising
// index), every token before which less than p of the probability lies; then one draw from the softmax of what is left:
// the first index whose running sum in index order exceeds u times the total. One block of 1024 threads per row.
// Nothing is sorted: the thresholds are found by radix selection over an order-preserving 32-bit key of the logit,
// eight passes of 4 bits, with a histogram of counts for top-k and of probability mass (float64) for top-p. Each thread
// fills 16 bins of its own in shared memory and the bins are then summed over the threads in a fixed order, so there
// are no atomics and the result is the same from run to run. exp(x / T - max) of every token is computed once, in
// float64, into `scratch` (V doubles per row); dropped tokens are zeroed there.
constexpr int SF_THREADS = 1024;
constexpr int SF_BINS = 16;
constexpr size_t SF_SMEM = (size_t)SF_BINS * SF_THREADS * sizeof(double);

__device__ __forceinline__ uint32_t falling_key(float x) {      // smaller key = larger value; -0 counts as +0
  const uint32_t u = __float_as_uint(x + 0.f);
  return ~((u & 0x80000000u) ? ~u : (u | 0x80000000u));
}

// Sum of v over the block in a fixed order; every thread gets it. s_part: 32 doubles.
__device__ __forceinline__ double block_sum_fixed(double v, double* s_part) {
  for (int o = 16; o; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = v;
  __syncthreads();
  double run = 0.0;
  for (int w = 0; w < SF_THREADS / 32; ++w) run += s_part[w];
  return run;
}

// bins[b * SF_THREADS + t]: thread t's share of bin b. Leaves the sums over the threads in total[0..15].
template <typename T>
__device__ __forceinline__ void sum_bins(const T* bins, T* s_part, T* total) {
  __syncthreads();
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31, b = w & (SF_BINS - 1), half = w >> 4;
  T acc = 0;
  for (int j = 0; j < SF_THREADS / 64; ++j) acc += bins[b * SF_THREADS + half * (SF_THREADS / 2) + j * 32 + lane];
  for (int o = 16; o; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
  if (lane == 0) s_part[w] = acc;
  __syncthreads();
  if (threadIdx.x < SF_BINS) total[threadIdx.x] = s_part[threadIdx.x] + s_part[threadIdx.x + SF_BINS];
  __syncthreads();
}

// f(i, key of row[i]) for every i this thread owns (i = tid, tid + 1024, ...), eight loads in flight at a time.
template <typename F>
__device__ __forceinline__ void for_each_key(const float* __restrict__ row, int V, F f) {
  constexpr int U = 8;
  for (int base = threadIdx.x; base < V; base += SF_THREADS * U) {
    float x[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + u * SF_THREADS;
      x[u] = i < V ? row[i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + u * SF_THREADS;
      if (i < V) f(i, x[u], falling_key(x[u]));
    }
  }
}

// Inclusive sum over the lanes below and this one, always in the same order.
__device__ __forceinline__ double warp_scan_fixed(double v, int lane) {
  for (int o = 1; o < 32; o <<= 1) {
    const double up = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += up;
  }
  return v;
}

__global__ void __launch_bounds__(SF_THREADS, 1)
sample_filtered_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                       const int* __restrict__ top_k, const float* __restrict__ top_p,
                       const double* __restrict__ uniform, double* __restrict__ scratch, int* __restrict__ out, int V) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  extern __shared__ __align__(16) unsigned char sf_smem[];
  double* bins_d = reinterpret_cast<double*>(sf_smem);
  unsigned int* bins_u = reinterpret_cast<unsigned int*>(sf_smem);
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ double s_part[32], s_mass[SF_BINS], s_wsum[32];
  __shared__ unsigned int s_partu[32], s_count[SF_BINS];
  __shared__ int s_wties[32];
  __shared__ uint32_t s_prefix;
  __shared__ unsigned int s_rank;
  __shared__ double s_need, s_target;
  __shared__ int s_res, s_warp;
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* row = logits + (size_t)r * V;
  double* e = scratch + (size_t)r * V;
  const float T = temperature[r];
  const int k = top_k[r];
  const int amax = block_argmax(row, V, s_val, s_idx);
  if (!(T > 0.f) || k == 1) {
    if (tid == 0) out[r] = amax;
    return;
  }
  const double mx = (double)row[amax] / (double)T;
  const uint32_t top_key = falling_key(row[amax]);
  // ---- top-k: the key of the k-th largest logit (x / T rises with x, so the selection runs on the logits themselves)
  uint32_t k_key = 0xffffffffu;                 // tokens with a key <= k_key stay
  if (k > 0 && k < V) {
    if (tid == 0) { s_prefix = 0u; s_rank = (unsigned int)(k - 1); }
    for (int pass = 0; pass < 8; ++pass) {
      const int shift = 28 - 4 * pass;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      for (int b = 0; b < SF_BINS; ++b) bins_u[b * SF_THREADS + tid] = 0u;
      for_each_key(row, V, [&](int, float, uint32_t key) {
        if (pass == 0 || (key >> (shift + 4)) == prefix) bins_u[((key >> shift) & 15u) * SF_THREADS + tid] += 1u;
      });
      sum_bins(bins_u, s_partu, s_count);
      if (tid == 0) {
        unsigned int rank = s_rank, cum = 0;
        int b = 0;
        for (; b < SF_BINS - 1; ++b) {
          if (cum + s_count[b] > rank) break;
          cum += s_count[b];
        }
        s_prefix = (prefix << 4) | (uint32_t)b;
        s_rank = rank - cum;
      }
    }
    __syncthreads();
    k_key = s_prefix;
  }
  // ---- top-p: the key of the last value of which something stays, and the mass that is still missing where it begins.
  // All keys that stay lie between top_key and k_key: the digits these two share are not searched. The first pass that
  // is searched also computes exp(x / T - max) of what top-k keeps, and the sum.
  const float pp = top_p[r];
  const bool nucleus = pp < 1.0f;
  const int first = nucleus ? __clz((int)(top_key ^ k_key)) / 4 : 8;       // 8: all digits shared, or no top-p
  uint32_t t_key = nucleus ? top_key : 0xffffffffu;                         // (first == 8: one value stays)
  double need_at_t = 0.0, total = 0.0;
  if (first == 8) {
    double local = 0.0;
    for_each_key(row, V, [&](int i, float x, uint32_t key) {
      const double v = key <= k_key ? exp((double)x / (double)T - mx) : 0.0;
      e[i] = v;
      local += v;
    });
    total = block_sum_fixed(local, s_part);
    need_at_t = (double)pp * total;
  } else {
    if (tid == 0) s_prefix = first == 0 ? 0u : top_key >> (32 - 4 * first);
    for (int pass = first; pass < 8; ++pass) {
      const int shift = 28 - 4 * pass;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      for (int b = 0; b < SF_BINS; ++b) bins_d[b * SF_THREADS + tid] = 0.0;
      if (pass == first) {
        double local = 0.0;
        for_each_key(row, V, [&](int i, float x, uint32_t key) {
          const double v = key <= k_key ? exp((double)x / (double)T - mx) : 0.0;
          e[i] = v;
          local += v;
          if (key <= k_key) bins_d[((key >> shift) & 15u) * SF_THREADS + tid] += v;
        });
        total = block_sum_fixed(local, s_part);
        if (tid == 0) s_need = (double)pp * total;
      } else {
        for_each_key(row, V, [&](int i, float, uint32_t key) {
          if (key <= k_key && (key >> (shift + 4)) == prefix) bins_d[((key >> shift) & 15u) * SF_THREADS + tid] += e[i];
        });
      }
      sum_bins(bins_d, s_part, s_mass);
      if (tid == 0) {
        // bins run from the largest values down: the first one at whose end the mass reaches what is needed holds the
        // threshold; if rounding leaves the sum a hair short, the last bin with any mass does
        const double need = s_need;
        double cum = 0.0, cum_last = 0.0;
        int b = 0, last = 0;
        for (; b < SF_BINS; ++b) {
          if (s_mass[b] > 0.0) { last = b; cum_last = cum; }
          if (cum + s_mass[b] >= need) break;
          cum += s_mass[b];
        }
        if (b == SF_BINS) { b = last; cum = cum_last; }
        s_prefix = (prefix << 4) | (uint32_t)b;
        s_need = need - cum;
      }
    }
    __syncthreads();
    t_key = s_prefix;
    need_at_t = s_need;
  }
  // ---- the draw. Warp w owns the contiguous range [w * span, (w + 1) * span) and walks it 32 tokens at a time, so that
  // sums run in index order. Equal values at the threshold: the j-th of them in index order (j = 0, 1, ...) stays while
  // j * e < need_at_t.
  const int span = ((V + 1023) / 1024) * 32;
  const int w_lo = min(V, warp * span), w_hi = min(V, w_lo + span);
  if (nucleus) {
    int ties = 0;
    for (int i = w_lo + lane; i < w_hi; i += 32) ties += falling_key(row[i]) == t_key ? 1 : 0;
    for (int o = 16; o; o >>= 1) ties += __shfl_xor_sync(0xffffffffu, ties, o);
    if (lane == 0) s_wties[warp] = ties;
  }
  __syncthreads();
  int j0 = 0;
  if (nucleus)
    for (int w = 0; w < warp; ++w) j0 += s_wties[w];
  double run = 0.0;
  for (int base = w_lo; base < w_hi; base += 32) {
    const int i = base + lane;
    const bool in = i < w_hi;
    double v = in ? e[i] : 0.0;
    if (nucleus) {
      const uint32_t key = in ? falling_key(row[i]) : 0u;
      const bool tie = in && key == t_key;
      const unsigned int tie_mask = __ballot_sync(0xffffffffu, tie);
      bool drop = in && key > t_key;
      if (tie) drop = !((double)(j0 + __popc(tie_mask & ((1u << lane) - 1u))) * v < need_at_t);
      j0 += __popc(tie_mask);
      if (drop && v != 0.0) e[i] = 0.0;
      if (drop) v = 0.0;
    }
    run += __shfl_sync(0xffffffffu, warp_scan_fixed(v, lane), 31);
  }
  if (lane == 0) s_wsum[warp] = run;
  __syncthreads();
  if (tid == 0) {
    double before = 0.0;
    for (int w = 0; w < 32; ++w) before += s_wsum[w];
    const double target = uniform[r] * before;
    before = 0.0;
    int w = 0;
    for (; w < 31; ++w) {
      if (before + s_wsum[w] > target) break;
      before += s_wsum[w];
    }
    s_warp = w;
    s_need = before;
    s_target = target;
    s_res = amax;   // stays only if rounding leaves every running sum at or below the target
  }
  __syncthreads();
  if (warp == s_warp) {
    const double target = s_target;
    run = s_need;
    for (int base = w_lo; base < w_hi; base += 32) {
      const int i = base + lane;
      const double sc = warp_scan_fixed(i < w_hi ? e[i] : 0.0, lane);
      const unsigned int hit = __ballot_sync(0xffffffffu, run + sc > target);
      if (hit) {
        if (lane == 0) s_res = base + __ffs(hit) - 1;
        break;
      }
      run += __shfl_sync(0xffffffffu, sc, 31);
    }
  }
  __syncthreads();
  if (tid == 0) out[r] = s_res;
}

// scratch: R * V doubles. top_k[r] <= 0 or >= V: no top-k; top_p[r] >= 1: no top-p; temperature[r] <= 0 or top_k[r]
// == 1: argmax.
FZ_API int fz_sample_filtered(const float* logits, const float* temperature, const int* top_k, const float* top_p,
                              const double* uniform, double* scratch, int* out, int R, int V, cudaStream_t stream) {
  if (R <= 0) return FZ_OK;
  if (V <= 0) return FZ_BAD_SHAPE;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(sample_filtered_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SF_SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  fz_launch(sample_filtered_kernel, dim3(R), dim3(SF_THREADS), SF_SMEM, stream, logits, temperature, top_k, top_p, uniform,
            scratch, out, V);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

// ------------------------------------------------------------------------------------------------ error word
// The error word is a device int the caller owns; this clears it on a stream.
FZ_API int fz_clear_error(int* err, cudaStream_t stream) {
  return (int)cudaMemsetAsync(err, 0, sizeof(int), stream);
}

// ------------------------------------------------------------------------------------------------ argmax without allocation
// See no_alloc.h. The scratch of the row-split argmax sits in this fixed device array. In host code the array's name is
// only a stand-in for the symbol, not a device address, so the address is looked up once per device and passed to the
// kernel as a pointer.
#include "no_alloc.h"
#include <mutex>
#include <stdio.h>

static __device__ __align__(256) unsigned char fz_no_alloc_scratch[FZ_NO_ALLOC_SCRATCH_BYTES];
static_assert(FZ_NO_ALLOC_MAX_SLICES == FZ_ARGMAX_MAX_SLICES,
              "the fixed scratch is laid out for as many slices per row as the row-split argmax may use");

namespace {
constexpr int NO_ALLOC_MAX_DEVICES = 64;
void* g_no_alloc_ptr[NO_ALLOC_MAX_DEVICES] = {};
std::mutex g_no_alloc_mu;
thread_local char g_no_alloc_error[256] = "";

// The scratch array's address on the current device (looked up at the first call on that device).
int no_alloc_scratch(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    snprintf(g_no_alloc_error, sizeof g_no_alloc_error, "cudaGetDevice failed: %s", cudaGetErrorString(e));
    return (int)e;
  }
  if (dev < 0 || dev >= NO_ALLOC_MAX_DEVICES) {
    snprintf(g_no_alloc_error, sizeof g_no_alloc_error, "device ordinal %d is outside 0..%d", dev, NO_ALLOC_MAX_DEVICES - 1);
    return FZ_TOO_LARGE;
  }
  std::lock_guard<std::mutex> lock(g_no_alloc_mu);
  if (g_no_alloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, fz_no_alloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      snprintf(g_no_alloc_error, sizeof g_no_alloc_error, "cudaGetSymbolAddress failed on device %d: %s", dev,
               cudaGetErrorString(e));
      return e != cudaSuccess ? (int)e : FZ_BAD_ALIGNMENT;
    }
    g_no_alloc_ptr[dev] = p;
  }
  *out = g_no_alloc_ptr[dev];
  return FZ_OK;
}
}  // namespace

FZ_API const char* fz_no_alloc_last_error(void) { return g_no_alloc_error; }

FZ_API int fz_argmax_no_alloc(const float* logits, int* out, int rows, int vocab, cudaStream_t stream) {
  g_no_alloc_error[0] = 0;
  if (rows <= 0) return FZ_OK;
  if (vocab <= 0 || logits == nullptr || out == nullptr) {
    snprintf(g_no_alloc_error, sizeof g_no_alloc_error, "bad arguments: rows %d, vocab %d, logits %p, out %p", rows, vocab,
             (const void*)logits, (void*)out);
    return FZ_BAD_SHAPE;
  }
  if (rows > FZ_NO_ALLOC_MAX_ROWS) {
    snprintf(g_no_alloc_error, sizeof g_no_alloc_error,
             "%d rows exceed the fixed scratch of this entry point (at most %d rows per call); split the call", rows,
             FZ_NO_ALLOC_MAX_ROWS);
    return FZ_TOO_LARGE;
  }
  const int slices = fz_argmax_slices(vocab);
  if (slices > FZ_NO_ALLOC_MAX_SLICES) {      // cannot happen while the two limits are equal (asserted above)
    snprintf(g_no_alloc_error, sizeof g_no_alloc_error, "%d slices per row exceed the fixed scratch (at most %d)", slices,
             FZ_NO_ALLOC_MAX_SLICES);
    return FZ_TOO_LARGE;
  }
  void* base = nullptr;
  const int st = no_alloc_scratch(&base);
  if (st != FZ_OK) return st;
  // [partial values: MAX_ROWS x MAX_SLICES float][partial indices: the same in int][counters: MAX_ROWS int]
  float* partial_val = (float*)base;
  int* partial_idx = (int*)((unsigned char*)base + (size_t)FZ_NO_ALLOC_MAX_ROWS * FZ_NO_ALLOC_MAX_SLICES * 4);
  int* counters = (int*)((unsigned char*)base + (size_t)FZ_NO_ALLOC_MAX_ROWS * FZ_NO_ALLOC_MAX_SLICES * 8);
  // the counters must start at zero whatever an earlier call left behind
  cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)rows * sizeof(int), stream);
  if (e != cudaSuccess) {
    snprintf(g_no_alloc_error, sizeof g_no_alloc_error, "clearing the counters failed: %s", cudaGetErrorString(e));
    return (int)e;
  }
  dim3 grid(rows, slices);
  // launched without the dependent-launch attribute: the memset above must be complete before the kernel starts
  argmax_kernel<<<grid, 512, 0, stream>>>(logits, out, vocab, partial_val, partial_idx, counters);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(g_no_alloc_error, sizeof g_no_alloc_error, "the launch failed: %s", cudaGetErrorString(e));
    return (int)e;
  }
  return FZ_OK;
}

#ifdef FZ_TIMELINE
FZ_TIMELINE_READER(rowwise)
#endif
