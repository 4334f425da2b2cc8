// Paged attention for decoded tokens and short portions, bf16 cache, on tensor cores, split over key partitions.
//
// grid (partitions, kv heads, token rows), 128 threads. A CTA serves one token row, one kv head and one partition of
// PART = 256 consecutive key positions (partition i holds keys 256 i .. 256 i + 255, whatever the batch: a row's sums
// have one order that depends only on its own position). All G = Hq / Hkv query heads of the kv head are the rows of
// the 16-row MMA tile, so the keys and values of the partition are read once for the whole group (the reference's
// default decode kernel lays the group out the same way: fusezap/device/cuda_kernels/attention.py:860-1043).
// Keys and values come in tiles of 64 through a three-stage cp.async ring; warp w owns keys 16 w .. 16 w + 15 of each
// tile: S = Q K^T and O += P V with mma.sync m16n8k16, softmax online in the exp2 domain with float32 max and sum, P
// rounded to bf16 for the second product. The four warps' (max, sum, O) are merged in warp order, and the partition's
// unnormalised O with its (max, sum) goes to a float32 scratch; `attn_combine_kernel` merges a row's partitions in
// rising order and normalises. Rows of portions with at least `long_from` tokens are left to the prefill kernel.
#include "attn_mma.cuh"
#include <math.h>

namespace {
using namespace fzattn;

constexpr int PART = 256;      // keys per partition
constexpr int TILE = 64;       // keys per shared-memory tile
constexpr int THREADS = 128;
constexpr int STAGES = 3;      // key / value tiles in flight

template <int HD>
__global__ void __launch_bounds__(THREADS)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                   const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ pos,
                   const int* __restrict__ seq_row, const int* __restrict__ seg, const int* __restrict__ table, int mb,
                   long long page_stride, int page_size, float* __restrict__ part_o, float* __restrict__ part_ml,
                   int Hq, int Hkv, float scale_log2, int window, int long_from) {
  fz_grid_wait();
  fz_grid_launch_dependents();
  constexpr int KSTEPS = HD / 16;      // k-steps of Q K^T
  constexpr int NB = HD / 8;           // 8-wide output blocks of P V
  extern __shared__ __align__(128) uint8_t smem[];
  // [STAGES][K tile | V tile] then the Q tile; the merge buffers reuse the stages
  constexpr int TILE_BYTES = TILE * HD * 2;
  const uint32_t s_base = smem_u32(smem);
  const uint32_t s_q = s_base + 2 * STAGES * TILE_BYTES;

  const int part = blockIdx.x, kvh = blockIdx.y, n = blockIdx.z, NP = gridDim.x;
  const int G = Hq / Hkv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = seq_row[n];
  if (row < 0) return;
  if (seg[row * 4 + 1] >= long_from) return;      // a long portion: the prefill kernel's rows
  const int p = pos[n];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int k_begin = max(part * PART, lo & ~(TILE - 1)), k_end = min((part + 1) * PART, p + 1);   // [k_begin, k_end)
  float* ml_out = part_ml + (((size_t)n * Hq + (size_t)kvh * G) * NP + part) * 2;
  if (k_begin >= k_end) {   // nothing of this row in this partition
    for (int g = tid; g < G; g += THREADS) { ml_out[(size_t)g * NP * 2] = -INFINITY; ml_out[(size_t)g * NP * 2 + 1] = 0.f; }
    return;
  }
  const int* trow = table + (size_t)row * mb;
  const long long head_off = (long long)kvh * page_size * HD;

  // Q: G rows of HD, zero rows up to 16, swizzled
  {
    const __nv_bfloat16* qrow = q + (size_t)n * Hq * HD + (size_t)kvh * G * HD;
    for (int e = tid; e < 16 * (HD / 8); e += THREADS) {
      const int r = e / (HD / 8), c = e - r * (HD / 8);
      cp_async16(s_q + swz<HD>(r, c), qrow + (size_t)r * HD + c * 8, r < G);
    }
  }
  const int ntiles = (k_end - k_begin + TILE - 1) / TILE;
  auto issue = [&](int t) {      // one commit group per call, empty past the last tile
    if (t < ntiles) {
      const uint32_t st = s_base + (t % STAGES) * 2 * TILE_BYTES;
      load_kv_tile<HD, TILE, THREADS>(st, st + TILE_BYTES, k_pool, v_pool, trow, page_stride, head_off, page_size,
                                      k_begin + t * TILE, lo, p, tid);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int t = 0; t < STAGES - 1; ++t) issue(t);

  uint32_t qf[KSTEPS][4];
  float o[NB][4];
#pragma unroll
  for (int i = 0; i < NB; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // rows lane/4 and lane/4 + 8

  for (int t = 0; t < ntiles; ++t) {
    issue(t + STAGES - 1);
    cp_async_wait<STAGES - 1>();      // all but the newest STAGES - 1 groups have landed: tile t is in
    __syncthreads();
    if (t == 0) {
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks)
        ldmatrix_x4(qf[ks], s_q + swz<HD>(lane & 15, ks * 2 + (lane >> 4)));
    }
    const uint32_t sk = s_base + (t % STAGES) * 2 * TILE_BYTES, sv = sk + TILE_BYTES;
    // S (16 x 16): this warp's keys 16 warp .. + 15 of the tile
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      uint32_t kf[4];
      const int mi = lane >> 3;
      ldmatrix_x4(kf, sk + swz<HD>(warp * 16 + (mi >> 1) * 8 + (lane & 7), ks * 2 + (mi & 1)));
      mma_bf16(s[0], qf[ks], kf[0], kf[1]);
      mma_bf16(s[1], qf[ks], kf[2], kf[3]);
    }
    const int key_base = k_begin + t * TILE + warp * 16 + 2 * (lane & 3);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key_base + 8 * j + (e & 1);
        const bool valid = key >= lo && key <= p;
        s[j][e] = valid ? s[j][e] * scale_log2 : -INFINITY;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
      }
    uint32_t pf[4];
    float corr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float mn = fmaxf(m_run[h], mx[h]);
      const float mu = mn == -INFINITY ? 0.f : mn;      // no visible key yet: every exponent below is exp2(-inf) = 0
      corr[h] = exp2f(m_run[h] - mu);
      m_run[h] = mn;
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float e0 = exp2f(s[j][2 * h] - mu), e1 = exp2f(s[j][2 * h + 1] - mu);
        sum += e0 + e1;
        pf[2 * j + h] = pack_bf16(e0, e1);
      }
      l_run[h] = l_run[h] * corr[h] + sum;
    }
#pragma unroll
    for (int i = 0; i < NB; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
    // O (16 x HD) += P (16 x 16) V (16 x HD)
#pragma unroll
    for (int nb = 0; nb < NB; nb += 2) {
      uint32_t vf[4];
      const int mi = lane >> 3;
      ldmatrix_x4_trans(vf, sv + swz<HD>(warp * 16 + (mi & 1) * 8 + (lane & 7), nb + (mi >> 1)));
      mma_bf16(o[nb], pf, vf[0], vf[1]);
      mma_bf16(o[nb + 1], pf, vf[2], vf[3]);
    }
    __syncthreads();   // the stage may be refilled
  }
  // ---- merge the four warps in warp order; rows g < G only
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  float* m_o = (float*)smem;                        // [4 warps][16 rows][HD]
  float* m_ml = m_o + 4 * 16 * HD;                  // [4][16][2]
  const int r0 = lane >> 2;
#pragma unroll
  for (int i = 0; i < NB; ++i) {
    const int d = 8 * i + 2 * (lane & 3);
    float* w0 = m_o + ((size_t)warp * 16 + r0) * HD + d;
    w0[0] = o[i][0]; w0[1] = o[i][1];
    w0[8 * HD] = o[i][2]; w0[8 * HD + 1] = o[i][3];
  }
  if ((lane & 3) == 0) {
    m_ml[(warp * 16 + r0) * 2] = m_run[0]; m_ml[(warp * 16 + r0) * 2 + 1] = l_run[0];
    m_ml[(warp * 16 + r0 + 8) * 2] = m_run[1]; m_ml[(warp * 16 + r0 + 8) * 2 + 1] = l_run[1];
  }
  __syncthreads();
  for (int e = tid; e < G * HD; e += THREADS) {
    const int g = e / HD, d = e - g * HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, m_ml[(w * 16 + g) * 2]);
    const float Mu = M == -INFINITY ? 0.f : M;
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(m_ml[(w * 16 + g) * 2] - Mu);
      acc += m_o[((size_t)w * 16 + g) * HD + d] * f;
      L += m_ml[(w * 16 + g) * 2 + 1] * f;
    }
    part_o[(((size_t)n * Hq + (size_t)kvh * G + g) * NP + part) * HD + d] = acc;
    if (d == 0) { ml_out[(size_t)g * NP * 2] = M; ml_out[(size_t)g * NP * 2 + 1] = L; }
  }
}

// One block per (token row, query head): merges the partitions in rising order, normalises, rounds to bf16.
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const int* __restrict__ seq_row, const int* __restrict__ seg,
                                    __nv_bfloat16* __restrict__ out, int Hq, int HD, int NP, int long_from) {
  fz_grid_wait();
  fz_grid_launch_dependents();
  const int n = blockIdx.y, h = blockIdx.x;
  __nv_bfloat16* orow = out + ((size_t)n * Hq + h) * HD;
  const int row = seq_row[n];
  if (row < 0) {
    for (int d = threadIdx.x; d < HD; d += blockDim.x) orow[d] = __float2bfloat16_rn(0.f);
    return;
  }
  if (seg[row * 4 + 1] >= long_from) return;
  const float* ml = part_ml + ((size_t)n * Hq + h) * NP * 2;
  const float* po = part_o + ((size_t)n * Hq + h) * NP * HD;
  float M = -INFINITY;
  for (int i = 0; i < NP; ++i) M = fmaxf(M, ml[2 * i]);
  float L = 0.f;
  for (int i = 0; i < NP; ++i) L += ml[2 * i + 1] * exp2f(ml[2 * i] - M);
  const float inv = 1.0f / L;
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float acc = 0.f;
    for (int i = 0; i < NP; ++i) {
      const float f = exp2f(ml[2 * i] - M);
      if (f != 0.f) acc += po[(size_t)i * HD + d] * f;     // an empty partition's O was never written
    }
    orow[d] = __float2bfloat16_rn(acc * inv);
  }
}

template <int HD>
int launch(const void* q, const void* k_pool, const void* v_pool, const int* pos, const int* seq_row, const int* seg,
           const int* table, int mb, long long page_stride, int page_size, void* out, float* part_o, float* part_ml,
           int N, int Hq, int Hkv, float scale, int window, int NP, int long_from, cudaStream_t stream) {
  constexpr int TILE_BYTES = TILE * HD * 2;
  constexpr size_t smem_pipe = 2 * STAGES * TILE_BYTES + 16 * HD * 2;
  constexpr size_t smem_merge = (size_t)4 * 16 * HD * 4 + 4 * 16 * 2 * 4;
  constexpr size_t smem = smem_pipe > smem_merge ? smem_pipe : smem_merge;
  static bool raised = false;
  if (smem > 48 * 1024 && !raised) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    raised = true;
  }
  dim3 grid(NP, Hkv, N);
  fz_launch(attn_decode_kernel<HD>, grid, dim3(THREADS), smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool,
            (const __nv_bfloat16*)v_pool, pos, seq_row, seg, table, mb, page_stride, page_size, part_o, part_ml, Hq, Hkv,
            scale * 1.4426950408889634f, window, long_from);
  FZ_LAUNCH_CHECK();
  dim3 cgrid(Hq, N);
  fz_launch(attn_combine_kernel, cgrid, dim3(HD < 128 ? 64 : 128), 0, stream, (const float*)part_o, (const float*)part_ml,
            seq_row, seg, (__nv_bfloat16*)out, Hq, HD, NP, long_from);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}
}  // namespace

// Sizes this kernel takes: head_dim 64 or 128, Hq / Hkv <= 16. Anything else is refused (the general kernel takes it).
FZ_API int fz_attn_decode_check(int Hq, int Hkv, int hd) {
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || Hq / Hkv > 16) return FZ_BAD_SHAPE;
  if (hd != 64 && hd != 128) return FZ_BAD_SHAPE;
  return FZ_OK;
}

FZ_API int fz_attn_partitions(int max_context) { return max_context <= 0 ? 1 : (max_context + PART - 1) / PART; }

// Float32 scratch the call needs: part_o N * Hq * NP * hd floats, part_ml N * Hq * NP * 2 floats.
FZ_API int fz_attn_decode(const void* q, const void* k_pool, const void* v_pool, const int* pos, const int* seq_row,
                          const int* seg, const int* table, int mb, long long page_stride, int page_size, void* out,
                          float* part_o, float* part_ml, int N, int Hq, int Hkv, int hd, float scale, int window,
                          int max_context, int long_from, cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (fz_attn_decode_check(Hq, Hkv, hd) != FZ_OK || page_size <= 0) return FZ_BAD_SHAPE;
  if (N > 65535 || Hkv > 65535) return FZ_TOO_LARGE;
  const int NP = fz_attn_partitions(max_context);
  if (hd == 64)
    return launch<64>(q, k_pool, v_pool, pos, seq_row, seg, table, mb, page_stride, page_size, out, part_o, part_ml, N, Hq, Hkv, scale, window, NP, long_from, stream);
  return launch<128>(q, k_pool, v_pool, pos, seq_row, seg, table, mb, page_stride, page_size, out, part_o, part_ml, N, Hq, Hkv, scale, window, NP, long_from, stream);
}
